// Dense core of a NORMALISED adjacency block as an exact small-integer matrix on the bf16 tensor-core path.
//
// The values of a symmetrically normalised adjacency matrix factor: val[r, c] = d_row[r] * (cnt[r, c] * d_col[c])
// with cnt the multiplicity of the edge (1 in a simple graph) and d = degree^-1/2 (gcn_distr.py:412-470).  The dense
// hub-by-hub rectangle of such a block is therefore
//        core = diag(rs) . Cnt . diag(cs),        Cnt a matrix of small non-negative integers,
// and integers up to 256 are EXACT in bf16.  So
//        core . Bs = diag(rs) . ( Cnt . Y ),      Y = diag(cs) . Bs   (fp32),
// and only Y has to be split for the tensor cores: Y = y1 + y2 + y3, three bf16 terms that carry 24 significant
// bits between them; Cnt needs no split at all.  Against the 3xTF32 form (core_gemm_tc.cu: both operands split,
// three TF32 products) this is three bf16 products at twice the tensor rate from ONE stored operand of 2 bytes per
// cell instead of two of 4 bytes: about a third of the time and a quarter of the memory, which moves the density
// above which a dense cell beats a gathered nonzero from 9 % to about 2 %.
//
//   gather_scale_split3_kernel   Ys[k] = [y1 | y2 | y3] of cs[k] * B[idx[k], :]            (bf16, K x 3 half)
//   CUTLASS sm100 TMA + tcgen05.mma (kind::f16, bf16 in, fp32 accumulators in TMEM) in k chunks:
//                                D (+)= Cnt[:, k0:k0+kc) . Ys[k0:k0+kc)                     (fp32, R x 3 half)
//   add_rows_scaled3_kernel      C[rows[i], n] += rs[i] * (D[i, n] + (D[i, half+n] + D[i, 2 half+n]))
//
// The k range may be cut into chunks ("core_chunk_int") whose GEMMs add into D in their epilogue, a proper fp32
// addition; a tensor-core accumulator is not a round-to-nearest fp32 sum.  Every product Cnt * y is exact here, so
// the only roundings are those of the accumulations, and the error grows far more slowly with the chunk length than
// in the TF32 path (measured on a 30,720^2 core against fp64, largest error over largest magnitude: chunks of 1,024
// 1.1e-7, 2,048 1.1e-7, 4,096 1.4e-7, 8,192 2.1e-7, the whole range in one 6.3e-7), while every chunk costs a read
// and a write of the 224 MB scratch matrix (core multiply 4.17 / 3.37 / 3.04 / 3.04 / 2.90 ms).  The default, 32,768,
// is the largest side a core may have: one GEMM per multiply, 160 times inside the 1e-4 the results must meet.
//
// This file instantiates CUTLASS / CuTe templates (header tree found at build time) and adds the kernels around
// them.  Without the header tree the multiply reports CAGNET_E_ARG and the host layer keeps the other core kernels.
#include <cuda_bf16.h>

#include "common.cuh"

namespace cagnet {

// x = y1 + y2 + y3 up to 2^-24 relative: successive bf16 roundings of the remainder (each subtraction is exact).
__device__ __forceinline__ void split3_bf16(float x, __nv_bfloat16& a, __nv_bfloat16& b, __nv_bfloat16& c) {
  a = __float2bfloat16_rn(x);
  const float r1 = x - __bfloat162float(a);
  b = __float2bfloat16_rn(r1);
  const float r2 = r1 - __bfloat162float(b);
  c = __float2bfloat16_rn(r2);
}

// One thread per 8 columns of a gathered row (two 128-bit loads, three 128-bit stores).
__global__ void __launch_bounds__(256)
gather_scale_split3_kernel(const float* __restrict__ B, int64_t ldb, const int* __restrict__ idx,
                           const float* __restrict__ cs, int K, int f, __nv_bfloat16* __restrict__ out, int64_t half) {
  const int vecs = static_cast<int>(half / 8);
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= static_cast<int64_t>(K) * vecs) return;
  const int k = static_cast<int>(t / vecs), n = static_cast<int>(t % vecs) * 8;
  const float s = __ldg(cs + k);
  const float* row = B + static_cast<int64_t>(__ldg(idx + k)) * ldb;
  float v[8];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
    if (n + 4 * h < f) q = __ldg(reinterpret_cast<const float4*>(row + n + 4 * h));   // rows are padded to 4 floats
    v[4 * h + 0] = q.x; v[4 * h + 1] = q.y; v[4 * h + 2] = q.z; v[4 * h + 3] = q.w;
  }
  __align__(16) __nv_bfloat16 y[3][8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float x = (n + j < f) ? s * v[j] : 0.f;
    split3_bf16(x, y[0][j], y[1][j], y[2][j]);
  }
  __nv_bfloat16* o = out + static_cast<int64_t>(k) * 3 * half + n;
#pragma unroll
  for (int part = 0; part < 3; ++part)
    *reinterpret_cast<uint4*>(o + part * half) = *reinterpret_cast<const uint4*>(y[part]);
}

// One thread per float4 of an output row; the two small terms are added to each other first.
__global__ void __launch_bounds__(256)
add_rows_scaled3_kernel(const float* __restrict__ D, int64_t half, const int* __restrict__ rows,
                        const float* __restrict__ rs, int R, float* __restrict__ C, int64_t ldc, int f) {
  const int vecs = static_cast<int>(half / 4);
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= static_cast<int64_t>(R) * vecs) return;
  const int m = static_cast<int>(t / vecs), n = static_cast<int>(t % vecs) * 4;
  if (n >= f) return;
  const float* d = D + static_cast<int64_t>(m) * 3 * half + n;
  const float4 a = __ldg(reinterpret_cast<const float4*>(d));
  const float4 b = __ldg(reinterpret_cast<const float4*>(d + half));
  const float4 c = __ldg(reinterpret_cast<const float4*>(d + 2 * half));
  const float s = __ldg(rs + m);
  float* out = C + static_cast<int64_t>(__ldg(rows + m)) * ldc + n;
  if (n + 0 < f) out[0] += s * (a.x + (b.x + c.x));
  if (n + 1 < f) out[1] += s * (a.y + (b.y + c.y));
  if (n + 2 < f) out[2] += s * (a.z + (b.z + c.z));
  if (n + 3 < f) out[3] += s * (a.w + (b.w + c.w));
}

static int g_core_chunk_int = 32768;
int core_chunk_int() { return g_core_chunk_int; }
int set_core_chunk_int(int value) {
  if (value < 256 || value % 64) return 1;
  g_core_chunk_int = value;
  return 0;
}

}  // namespace cagnet

#ifdef CAGNET_HAVE_CUTLASS

#include "cute/tensor.hpp"
#include "cutlass/bfloat16.h"
#include "cutlass/cutlass.h"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/epilogue/thread/linear_combination.h"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/dispatch_policy.hpp"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/util/packed_stride.hpp"

namespace cagnet {
namespace tci {

using namespace cute;

using Element = cutlass::bfloat16_t;
using LayoutA = cutlass::layout::RowMajor;      // Cnt: R x K, k contiguous
using LayoutB = cutlass::layout::RowMajor;      // [y1 | y2 | y3]: K x N, n contiguous
using LayoutC = cutlass::layout::RowMajor;
constexpr int kAlignAB = 8;                     // 16-byte rows for TMA
constexpr int kAlignC = 4;

// One SM per 128 x 256 tile, cluster 1 x 1 x 1: every CTA loads its own operand tiles, nothing is shared between
// CTAs.  (A pair of SMs per 256 x 256 tile measured 16 % faster on one GPU, 2.74 against 3.27 ms for a 30,720^2
// core, but needs a 2 x 1 x 1 cluster; this library keeps every kernel it may run beside NCCL free of clusters.)
using MmaTile = Shape<_128, _256, _64>;
using Cluster = Shape<_1, _1, _1>;

using Epilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, MmaTile, Cluster,
    cutlass::epilogue::collective::EpilogueTileAuto, float, float, float, LayoutC, kAlignC, float, LayoutC, kAlignC,
    cutlass::epilogue::collective::EpilogueScheduleAuto>::CollectiveOp;

using Mainloop = typename cutlass::gemm::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, Element, LayoutA, kAlignAB, Element, LayoutB, kAlignAB, float,
    MmaTile, Cluster,
    cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epilogue::SharedStorage))>,
    cutlass::gemm::collective::KernelScheduleAuto>::CollectiveOp;

using Kernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, Mainloop, Epilogue>;
using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;

static typename Gemm::Arguments make_args(const Element* A, int64_t lda, const Element* B, int64_t ldb, float* D,
                                          int64_t ldd, int M, int N, int K, float beta) {
  using StrideA = typename Kernel::StrideA;
  using StrideB = typename Kernel::StrideB;
  using StrideC = typename Kernel::StrideC;
  using StrideD = typename Kernel::StrideD;
  StrideA sa = cutlass::make_cute_packed_stride(StrideA{}, cute::make_shape(M, K, 1));
  StrideB sb = cutlass::make_cute_packed_stride(StrideB{}, cute::make_shape(N, K, 1));
  StrideC sc = cutlass::make_cute_packed_stride(StrideC{}, cute::make_shape(M, N, 1));
  StrideD sd = cutlass::make_cute_packed_stride(StrideD{}, cute::make_shape(M, N, 1));
  // leading dimensions of the padded layouts (the packed helpers assume ld == extent)
  cute::get<0>(sa) = lda;
  cute::get<1>(sb) = ldb;
  cute::get<0>(sc) = ldd;
  cute::get<0>(sd) = ldd;
  return typename Gemm::Arguments{cutlass::gemm::GemmUniversalMode::kGemm,
                                  {M, N, K, 1},
                                  {A, sa, B, sb},
                                  {{1.0f, beta}, D, sc, D, sd}};
}

static int gemm(const Element* A, int64_t lda, const Element* B, int64_t ldb, float* D, int64_t ldd, int M, int N,
                int K, float beta, void* ws, size_t ws_bytes, cudaStream_t stream) {
  auto args = make_args(A, lda, B, ldb, D, ldd, M, N, K, beta);
  if (Gemm::get_workspace_size(args) > ws_bytes)
    return fail(CAGNET_E_WORKSPACE, "cagnet_core_gemm_int_bf16: workspace too small");
  Gemm op;
  if (op.can_implement(args) != cutlass::Status::kSuccess)
    return fail(CAGNET_E_ARG, "cagnet_core_gemm_int_bf16: shape or alignment not supported by the tensor-core mainloop");
  if (op.initialize(args, ws, stream) != cutlass::Status::kSuccess)
    return fail(CAGNET_E_LAUNCH, "cagnet_core_gemm_int_bf16: initialisation of the tensor-core multiply failed");
  if (op.run(stream) != cutlass::Status::kSuccess)
    return fail(CAGNET_E_LAUNCH, "cagnet_core_gemm_int_bf16: launch of the tensor-core multiply failed");
  return CAGNET_OK;
}

}  // namespace tci
}  // namespace cagnet

using namespace cagnet;

extern "C" int cagnet_core_gemm_int_available(void) { return 1; }

extern "C" size_t cagnet_core_gemm_int_workspace_bytes(int32_t R, int32_t K, int32_t f) {
  if (R <= 0 || K <= 0 || f <= 0) return 0;
  const int half = (f + 7) / 8 * 8;
  auto args = tci::make_args(nullptr, K, nullptr, 3 * half, nullptr, 3 * half, R, 3 * half,
                             K < core_chunk_int() ? K : core_chunk_int(), 0.f);
  return tci::Gemm::get_workspace_size(args) + 16;
}

extern "C" int cagnet_core_gemm_int_bf16(const void* cnt, int64_t ld_cnt, int32_t R, int32_t K, const void* Ys,
                                         int64_t half, float* D, int32_t f, void* ws, size_t ws_bytes, void* stream) {
  if (R < 0 || K < 0 || f < 0) return fail(CAGNET_E_ARG, "cagnet_core_gemm_int_bf16: negative size");
  if (R == 0 || K == 0 || f == 0) return CAGNET_OK;
  if (!cnt || !Ys || !D) return fail(CAGNET_E_ARG, "cagnet_core_gemm_int_bf16: null pointer");
  if (ld_cnt < K || half < f) return fail(CAGNET_E_ARG, "cagnet_core_gemm_int_bf16: leading dimension too small");
  if (ld_cnt % 8 || half % 8 || !aligned(cnt, 16) || !aligned(Ys, 16) || !aligned(D, 16))
    return fail(CAGNET_E_ALIGN, "cagnet_core_gemm_int_bf16: rows of Cnt, Ys and D must start on 16-byte boundaries");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const auto* A = static_cast<const tci::Element*>(cnt);
  const auto* Bm = static_cast<const tci::Element*>(Ys);
  const int N = static_cast<int>(3 * half);
  const int chunk = core_chunk_int();
  for (int k0 = 0; k0 < K; k0 += chunk) {
    const int kc = (K - k0 < chunk) ? K - k0 : chunk;
    const int rc = tci::gemm(A + k0, ld_cnt, Bm + static_cast<int64_t>(k0) * N, N, D, N, R, N, kc, k0 == 0 ? 0.f : 1.f,
                             ws, ws_bytes, s);
    if (rc) return rc;
  }
  return check_launch("cagnet_core_gemm_int_bf16");
}

#else  // no CUTLASS header tree at build time

using namespace cagnet;

extern "C" int cagnet_core_gemm_int_available(void) { return 0; }
extern "C" size_t cagnet_core_gemm_int_workspace_bytes(int32_t, int32_t, int32_t) { return 0; }
extern "C" int cagnet_core_gemm_int_bf16(const void*, int64_t, int32_t, int32_t, const void*, int64_t, float*, int32_t,
                                         void*, size_t, void*) {
  return fail(CAGNET_E_ARG, "cagnet_core_gemm_int_bf16: built without the CUTLASS header tree");
}

#endif

extern "C" int cagnet_gather_scale_split3_bf16(const float* B, int64_t ldb, const int32_t* idx, const float* cs,
                                               int32_t K, int32_t f, void* out, int64_t half, void* stream) {
  if (K < 0 || f < 0) return fail(CAGNET_E_ARG, "cagnet_gather_scale_split3_bf16: negative size");
  if (K == 0 || f == 0) return CAGNET_OK;
  if (!B || !idx || !cs || !out) return fail(CAGNET_E_ARG, "cagnet_gather_scale_split3_bf16: null pointer");
  const int64_t f4 = (static_cast<int64_t>(f) + 3) / 4 * 4, f8 = (static_cast<int64_t>(f) + 7) / 8 * 8;
  if (ldb < f4 || half < f8 || ldb % 4 || half % 8 || !aligned(B, 16) || !aligned(out, 16))
    return fail(CAGNET_E_ALIGN, "cagnet_gather_scale_split3_bf16: B rows padded to 4 floats, output rows to 8 elements, both 16-byte aligned");
  const int64_t threads = static_cast<int64_t>(K) * (half / 8);
  gather_scale_split3_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      B, ldb, idx, cs, K, f, static_cast<__nv_bfloat16*>(out), half);
  return check_launch("cagnet_gather_scale_split3_bf16");
}

extern "C" int cagnet_add_rows_scaled3_f32(const float* D, int64_t half, const int32_t* rows, const float* rs, int32_t R,
                                           int32_t f, float* C, int64_t ldc, void* stream) {
  if (R < 0 || f < 0) return fail(CAGNET_E_ARG, "cagnet_add_rows_scaled3_f32: negative size");
  if (R == 0 || f == 0) return CAGNET_OK;
  if (!D || !rows || !rs || !C) return fail(CAGNET_E_ARG, "cagnet_add_rows_scaled3_f32: null pointer");
  if (half < f || ldc < f || half % 4 || !aligned(D, 16))
    return fail(CAGNET_E_ALIGN, "cagnet_add_rows_scaled3_f32: D rows must be padded to a multiple of 4 floats and 16-byte aligned");
  const int64_t threads = static_cast<int64_t>(R) * (half / 4);
  add_rows_scaled3_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      D, half, rows, rs, R, C, ldc, f);
  return check_launch("cagnet_add_rows_scaled3_f32");
}
