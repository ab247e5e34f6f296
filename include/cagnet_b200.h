/*
 * cagnet_b200 -- C ABI of the B200 (sm_100a) kernels behind CAGNET's full-batch GCN hot path.
 *
 * Plain pointers and sizes only: every pointer is a DEVICE pointer unless its comment says host,
 * every matrix is fp32 row-major with an explicit leading dimension (elements, not bytes), sparse
 * indices are int32, `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 * Nothing here allocates, frees or synchronises unless its comment says so: scratch memory is
 * passed in by the caller.  Every function returns 0 on success or one of the CAGNET_E_* codes;
 * cagnet_last_error_string() describes the last failure on the calling thread.
 *
 * The reference interface each entry point replaces is cited as file:line of PASSIONLab/CAGNET.
 */
#ifndef CAGNET_B200_H
#define CAGNET_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  CAGNET_OK = 0,
  CAGNET_E_ARG = 1,        /* null pointer, negative size, bad enum */
  CAGNET_E_ALIGN = 2,      /* leading dimension smaller than the width, or a misaligned pointer */
  CAGNET_E_OVERFLOW = 3,   /* a size does not fit the 32-bit index type of the kernels */
  CAGNET_E_LAUNCH = 4,     /* CUDA reported an error at launch */
  CAGNET_E_WORKSPACE = 5,  /* scratch buffer too small */
  CAGNET_E_INVALID = 6     /* device-side validation found malformed input */
};

/* Epilogues of cagnet_gemm_nn_f32. */
enum {
  CAGNET_EPI_NONE = 0,
  CAGNET_EPI_RELU = 1,         /* out = max(acc, 0)                         F.relu,        gcn_distr.py:287-288 */
  CAGNET_EPI_LOG_SOFTMAX = 2,  /* out = log_softmax(acc) per row (N <= 64)  F.log_softmax, gcn_distr.py:285-286 */
  CAGNET_EPI_RELU_MASK = 3,    /* out = aux > 0 ? acc : 0  (ReLU backward;  replaces autograd.grad at gcn_distr.py:312-322) */
  CAGNET_EPI_ACCUMULATE = 4    /* out += acc               (`z_loc += torch.mm(acol, brow)`, gcn_distr_2d.py:507) */
};

int cagnet_version(void);
const char* cagnet_last_error_string(void);

/* Tuning knobs, for sweeps (host-side global state; CAGNET_E_ARG for an unknown name or value):
 *   "spmm_tile"        vectors per feature tile; 0 = automatic, which also picks the two-vectors-per-lane mapping for
 *                      products of 5..16 vectors
 *   "spmm_rpb"         rows (warps) per thread block of the row kernels
 *   "spmm_long"        rows with more nonzeros than this are listed in the plan and processed by a whole thread block
 *   "spmm_long_narrow" a lower bound on that limit for products narrower than 128 columns (= "spmm_long" by default)
 *   "spmm_group_avg"   blocks with at most this many nonzeros per row on average run the lane-group kernel when B is
 *                      narrower than 128 columns; 0 = never
 *   "spmm_group_max"   rows up to this length are walked by one lane group there, longer ones by the whole warp
 *   "spmm_group_pool"  consecutive rows per warp there; 0 = automatic
 *   "spmm_deep"        1 = one-vector-per-lane products on such blocks issue their gathers in batches of 8
 *   "spmm_overlap"     1 = the row kernel may start under the tail of the hub-row kernel of the same multiply
 *                      (programmatic dependent launch); 0 serialises them
 *   "core_chunk"       k length of one tensor-core accumulation of the 3xTF32 dense-core multiply (multiple of 32)
 *   "core_chunk_int"   the same for the integer-core multiply (multiple of 64) */
int cagnet_set_param(const char* name, int value);
int cagnet_get_param(const char* name);

/* ---- COO row indices -> CSR row offsets: rowptr[i] = |{e : rows[e] < i}|, i in [0, n].
 * `rows` sorted ascending (a coalesced COO).  Bit-exact integer work.
 * Replaces cusparseXcoo2csr at sparse-extension/sparse_coo_tensor.cu:137-142. */
int cagnet_coo2csr_i32(const int32_t* rows, int64_t nnz, int32_t n, int32_t* rowptr, void* stream);

/* Device-side validation of a CSR block: rowptr monotone, rowptr[0]=0, rowptr[n]=nnz, columns in
 * [0, m) and, when the COO row indices the offsets were made from are passed (rows != NULL), rows in
 * [0, n) and sorted ascending.  Writes 0 (valid) or a reason code (1 rowptr[0], 2 rowptr[n],
 * 3 unsorted, 4 column range, 5 row range) to *status_dev (one int32 on the device); the caller
 * reads it back.  No counterpart in the reference, which never validates (sparse_coo_tensor.cu:43-54
 * skips even torch's checks). */
int cagnet_check_csr_i32(const int32_t* rowptr, const int32_t* col, const int32_t* rows, int32_t n, int32_t m,
                         int64_t nnz, int32_t* status_dev, void* stream);

/* ---- SpMM plan: lists the rows of a CSR block that are long enough to need a whole thread block.
 * Scratch layout is opaque; size it with cagnet_spmm_plan_bytes(n, nnz).  Build once per block
 * (the adjacency never changes), reuse for every multiply.  */
size_t cagnet_spmm_plan_bytes(int32_t n, int64_t nnz);
int cagnet_spmm_plan_i32(const int32_t* rowptr, int32_t n, int64_t nnz, void* plan, size_t plan_bytes, void* stream);

/* ---- C = beta*C + A*B.  A: n x m CSR (rowptr[n+1], col[nnz], val[nnz]); B: m x f, ldb; C: n x f, ldc.
 * beta is 0 (overwrite) or 1 (accumulate, the reference's in-place `C += A.B`).
 * `plan` may be NULL (every row is then processed by one warp).  If ldb and ldc are multiples of 4
 * (2) and B, C are 16-byte (8-byte) aligned the kernel moves 128-bit (64-bit) vectors; columns
 * [f, ld) of such padded rows of B and C may be read, and are never written: exactly n x f elements of C change,
 * as with the reference op, so C may be a column slice of a wider matrix.
 * Replaces cusparseSpMM(alpha=1, beta=1, CSRMM_ALG1) plus the row/column-major re-layouts around
 * it at sparse-extension/sparse_coo_tensor.cu:149-226. */
int cagnet_spmm_csr_f32(const int32_t* rowptr, const int32_t* col, const float* val,
                        int32_t n, int32_t m, int64_t nnz,
                        const float* B, int64_t ldb, float* C, int64_t ldc, int32_t f, float beta,
                        const void* plan, void* stream);

/* ---- The same multiply for callers that cannot allocate device memory (no counterpart in the reference,
 * whose op calls cudaMalloc twice per call: sparse_coo_tensor.cu:136, 213).  Meant for hosts where every byte
 * of the GPU already belongs to another allocator, so that cudaMalloc fails, or where the device-wide
 * synchronisation hidden in cudaMalloc/cudaFree is not acceptable inside the loop that calls this.  The
 * hub-row list is built, on `stream`, in a fixed 256 KB device array that is part of the library (each GPU
 * that loads the library holds it until the process exits), then the multiply runs exactly as
 * cagnet_spmm_csr_f32 does with a plan.  Nothing is allocated or freed, here or in anything it calls.
 *   - Limit: nnz <= cagnet_spmm_noalloc_max_nnz() (65,535 x the hub-row threshold: about 134 M at the default
 *     2048); beyond it the call returns CAGNET_E_WORKSPACE and does nothing.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current; `stream` must belong to it).  Under CUDA's lazy module loading that look-up is also the
 *     moment the library's device code and this array are loaded onto the GPU, so "allocates nothing" holds from
 *     the second call on: make one warm-up call per device at start-up, before any stream capture and before
 *     the other allocator takes the rest of the memory.
 *   - All calls share the one array and the array keeps the last call's list: each call resets it first, and
 *     two calls whose kernels can overlap on the GPU (different streams, different host threads) race on it.
 *     Serialise them, or use cagnet_spmm_csr_f32 with one plan per block. */
int64_t cagnet_spmm_noalloc_max_nnz(void);
int cagnet_spmm_csr_f32_noalloc(const int32_t* rowptr, const int32_t* col, const float* val,
                                int32_t n, int32_t m, int64_t nnz,
                                const float* B, int64_t ldb, float* C, int64_t ldc, int32_t f, float beta,
                                void* stream);

/* ---- Dense core of a sparse block: C[core_rows[i], 0:f) += sum_j core[i*ld_core + j] * B[core_cols[j], 0:f)
 * for i < R, j < K.  `core` is the R x K dense fp32 sub-block (zeros where the sparse block has no entry) of
 * the hub rows `core_rows` (distinct, ascending or not) and hub columns `core_cols` that the host layer cut out
 * of a CSR block; the remaining entries go through cagnet_spmm_csr_f32, which must be queued first when it
 * overwrites C (beta = 0).  fp32 FMAs in a fixed order.  B rows 16-byte aligned (ldb % 4 == 0).
 * The k range is cut into slices whose partial sums pass through `ws` (16-byte aligned, at least
 * cagnet_core_gemm_workspace_bytes(R, K, f) bytes, which may be 0) and are added up in slice order.
 * Part of the work cusparseScsrmm2 does at sparse-extension/sparse_coo_tensor.cu:198-226; the reference has
 * no such split. */
size_t cagnet_core_gemm_workspace_bytes(int32_t R, int32_t K, int32_t f);
int cagnet_core_gemm_f32(const float* core, int64_t ld_core, const int32_t* core_rows, int32_t R,
                         const int32_t* core_cols, int32_t K,
                         const float* B, int64_t ldb, float* C, int64_t ldc, int32_t f,
                         void* ws, size_t ws_bytes, void* stream);

/* ---- The same dense core on the tensor cores (tcgen05, kind::tf32) with fp32 accuracy ("3xTF32"): operands are
 * split into hi (rounded to TF32) + lo (exact remainder) and core*Bs ~ hi*hi + (hi*lo + lo*hi).
 *   cagnet_split_tf32_f32            hi[i], lo[i] of x[i]; run once on the core when the block is planned.
 *   cagnet_gather_split_rows_f32     out[k] = [hi(B[idx[k]]) | lo(B[idx[k]])], K rows of 2*half floats, half >= f
 *                                    rounded up to a multiple of 4 (columns [f, half) of both halves zeroed).
 *   cagnet_core_gemm_tc_f32          D[R x 3*half]: columns [0, half) = core_hi*Bs_hi, [half, 2 half) =
 *                                    core_hi*Bs_lo, [2 half, 3 half) = core_lo*Bs_hi; the k range is cut into
 *                                    chunks whose sums are added in fp32 (a tensor-core accumulator over the whole
 *                                    k range loses about 3e-5 at k = 13K).  ws: cagnet_core_gemm_tc_workspace_bytes.
 *   cagnet_add_rows3_f32             C[rows[i], n] += D[i, n] + (D[i, half+n] + D[i, 2 half+n]), n < f.
 * All row starts 16-byte aligned.  cagnet_core_gemm_tc_available() is 0 when the library was built without the
 * CUTLASS header tree; the multiply then returns CAGNET_E_ARG (the three small kernels work regardless).
 * No counterpart in the reference. */
int cagnet_core_gemm_tc_available(void);
size_t cagnet_core_gemm_tc_workspace_bytes(int32_t R, int32_t K, int32_t f);
int cagnet_split_tf32_f32(const float* x, int64_t count, float* hi, float* lo, void* stream);
int cagnet_gather_split_rows_f32(const float* B, int64_t ldb, const int32_t* idx, int32_t K, int32_t f, float* out,
                                 int64_t half, void* stream);
int cagnet_core_gemm_tc_f32(const float* core_hi, const float* core_lo, int64_t ld_core, int32_t R, int32_t K,
                            const float* Bs, int64_t half, float* D, int32_t f, void* ws, size_t ws_bytes,
                            void* stream);
int cagnet_add_rows3_f32(const float* D, int64_t half, const int32_t* rows, int32_t R, int32_t f, float* C,
                         int64_t ldc, void* stream);

/* ---- The dense core of a NORMALISED block as an exact integer matrix on the bf16 tensor-core path.  A symmetrically
 * normalised adjacency value factors as rs[row] * (cnt * cs[col]) with cnt the edge multiplicity
 * (scale_elements, gcn_distr.py:412-470), so the core is diag(rs) . Cnt . diag(cs) with Cnt small integers, exact in
 * bf16, and only Y = diag(cs) . B[core_cols] needs splitting (three bf16 terms carry 24 significant bits):
 *   cagnet_gather_scale_split3_bf16  out[k] = [y1 | y2 | y3] of cs[k] * B[idx[k], 0:f), K rows of 3*half bf16, half >= f
 *                                    rounded up to a multiple of 8 (columns [f, half) of every part zeroed).
 *   cagnet_core_gemm_int_bf16        D[R x 3*half] (fp32) = Cnt[R x K] (bf16, ld_cnt) . out, tcgen05 kind::f16 with
 *                                    fp32 accumulation, the k range cut into "core_chunk_int" pieces added in fp32.
 *                                    ws: cagnet_core_gemm_int_workspace_bytes.
 *   cagnet_add_rows_scaled3_f32      C[rows[i], n] += rs[i] * (D[i, n] + (D[i, half+n] + D[i, 2 half+n])), n < f.
 * All row starts 16-byte aligned.  cagnet_core_gemm_int_available() is 0 when the library was built without the
 * CUTLASS header tree; the multiply then returns CAGNET_E_ARG (the two small kernels work regardless).
 * No counterpart in the reference, which hands normalised values to cuSPARSE like any others
 * (sparse-extension/sparse_coo_tensor.cu:198-226). */
int cagnet_core_gemm_int_available(void);
size_t cagnet_core_gemm_int_workspace_bytes(int32_t R, int32_t K, int32_t f);
int cagnet_gather_scale_split3_bf16(const float* B, int64_t ldb, const int32_t* idx, const float* cs, int32_t K,
                                    int32_t f, void* out, int64_t half, void* stream);
int cagnet_core_gemm_int_bf16(const void* cnt, int64_t ld_cnt, int32_t R, int32_t K, const void* Ys, int64_t half,
                              float* D, int32_t f, void* ws, size_t ws_bytes, void* stream);
int cagnet_add_rows_scaled3_f32(const float* D, int64_t half, const int32_t* rows, const float* rs, int32_t R,
                                int32_t f, float* C, int64_t ldc, void* stream);

/* ---- Z = epilogue(X * W) for a tall X (n x K, ldx) and a small W.
 * transW = 0: W is K x N row-major (ldw);  transW = 1: W is N x K row-major (ldw) and is used
 * transposed (the `mm(ag, weight.t())` form).  aux (n x N, ldaux) is read by CAGNET_EPI_RELU_MASK only.
 * Replaces torch.mm at gcn_distr.py:275 and :330 and the activations at gcn_distr.py:284-294. */
int cagnet_gemm_nn_f32(const float* X, int64_t ldx, const float* W, int64_t ldw, int32_t transW,
                       float* Z, int64_t ldz, int64_t n, int32_t K, int32_t N,
                       int32_t epilogue, const float* aux, int64_t ldaux, void* stream);

/* ---- out (K x N, ldo) = beta*out + H^T * G for tall H (n x K, ldh) and G (n x N, ldg): the weight
 * gradient.  beta is 0 or 1.  Split over row chunks, partial products in `ws`, summed in chunk order
 * (deterministic).  Size ws with cagnet_gemm_tn_workspace_bytes.  Replaces torch.mm(inputs.t(), ag) at
 * gcn_distr.py:187 (outer_product2) and the accumulating `z_loc += torch.mm(acol, brow)` of the dense
 * SUMMA at gcn_distr_2d.py:276 (whose left operand is a transposed block). */
size_t cagnet_gemm_tn_workspace_bytes(int64_t n, int32_t K, int32_t N);
int cagnet_gemm_tn_f32(const float* H, int64_t ldh, const float* G, int64_t ldg,
                       float* out, int64_t ldo, int64_t n, int32_t K, int32_t N, float beta,
                       void* ws, size_t ws_bytes, void* stream);

/* ---- Elementwise / row-wise pieces, for callers that do not use the fused epilogues. */
int cagnet_relu_fwd_f32(const float* z, int64_t ldz, float* h, int64_t ldh, int64_t n, int32_t N, void* stream);
/* dz = h > 0 ? g : 0 */
int cagnet_relu_bwd_f32(const float* h, int64_t ldh, const float* g, int64_t ldg, float* dz, int64_t lddz,
                        int64_t n, int32_t N, void* stream);
int cagnet_log_softmax_fwd_f32(const float* z, int64_t ldz, float* logp, int64_t ldl, int64_t n, int32_t N, void* stream);
/* dz = g - exp(logp) * rowsum(g): the closed form of what gcn_distr.py:312-322 obtains by re-running
 * log_softmax under autograd. */
int cagnet_log_softmax_bwd_f32(const float* logp, int64_t ldl, const float* g, int64_t ldg, float* dz, int64_t lddz,
                               int64_t n, int32_t N, void* stream);

/* ---- Row-wise pieces of a log-softmax whose rows are split by columns over several processes
 * (dist_log_softmax, gcn_distr_2d.py:537-568): each process reduces its own columns, the per-row scalars
 * are combined by a collective between the calls.
 * cagnet_row_reduce_f32: out[row] = max_c z (mode 0) | sum_c z (mode 1) | sum_c exp(z - ref[row]) (mode 2).
 * cagnet_log_softmax_apply_f32: logp = z - row_max - log(row_sum).
 * cagnet_log_softmax_bwd_apply_f32: dz = g - exp(logp) * row_sum_g (replaces the gather of full rows and
 * the autograd call of dist_log_softmax2, gcn_distr_2d.py:570-645, 777-795). */
int cagnet_row_reduce_f32(const float* z, int64_t ldz, int64_t n, int32_t N, int32_t mode, const float* ref,
                          float* out, void* stream);
int cagnet_log_softmax_apply_f32(const float* z, int64_t ldz, const float* row_max, const float* row_sum,
                                 float* logp, int64_t ldl, int64_t n, int32_t N, void* stream);
int cagnet_log_softmax_bwd_apply_f32(const float* logp, int64_t ldl, const float* g, int64_t ldg,
                                     const float* row_sum_g, float* dz, int64_t lddz, int64_t n, int32_t N,
                                     void* stream);

/* ---- Masked NLL: loss = -(1/count) * sum_{i: mask[i]} logp[i, y[i]];  writes the scalar to
 * *loss_dev and, if grad != NULL, grad[i, j] = -scale/count at (i, y[i]) for masked rows, else 0
 * (all n x N entries are written).  Rows whose label lies outside [cls_lo, cls_hi) are skipped
 * (the class-column restriction of the 2D/3D loss, gcn_distr_2d.py:962-989); labels are rebased
 * by cls_lo.  count is supplied by the caller (number of rows the mean runs over).
 * ws: cagnet_nll_workspace_bytes(n).  Replaces F.nll_loss(outputs[mask], y[mask]) at
 * gcn_distr.py:356 and its autograd backward. */
size_t cagnet_nll_workspace_bytes(int64_t n);
int cagnet_nll_masked_f32(const float* logp, int64_t ldl, const int64_t* y, const uint8_t* mask,
                          int64_t n, int32_t N, int32_t cls_lo, int32_t cls_hi, float count, float scale,
                          float* loss_dev, float* grad, int64_t ldg, void* ws, size_t ws_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CAGNET_B200_H */
