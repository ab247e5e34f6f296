// Dense core of a power-law adjacency block on the 5th-generation tensor cores (tcgen05 / TMEM) of sm_100a.
//
// D = core[R x K] * Bs[K x f] with fp32 accuracy from TF32 tensor-core products ("3xTF32"): every operand is
// split once into hi = its value rounded to TF32's 11 significant bits and lo = the remainder (exact in fp32),
// and
//     core * Bs  ~  core_hi * Bs_hi  +  (core_hi * Bs_lo + core_lo * Bs_hi)          (lo * lo ~ 2^-22 is dropped).
// The core is static, so its split is made once when the block is planned; the hub columns' rows of B are
// gathered and split in one pass per multiply (gather_split_rows_kernel writes [Bs_hi | Bs_lo] side by side, so
// core_hi needs a single GEMM against both).  The GEMMs are CUTLASS's sm100 TMA + tcgen05.mma (kind::tf32)
// warp-specialised mainloop, instantiated here: 128 x 128 x 32 tiles, accumulators in TMEM, cluster shape
// 1 x 1 x 1 (every CTA loads its own tiles), 1-SM MMA.
//
// Accuracy: a tensor-core accumulator is not a round-to-nearest fp32 sum, and its error grows with the length of
// the contraction (measured 2.8e-5 of the largest magnitude at k = 13,312 in one piece).  The k range is
// therefore cut into chunks (tuning knob "core_chunk", 2,048 by default); each chunk's GEMM adds into D in its epilogue (beta = 1), which is a
// proper fp32 addition.
//
// This file instantiates CUTLASS / CuTe templates (header tree found at build time) and adds the split kernels
// around them.  Without the header tree it compiles to a stub that reports CAGNET_E_ARG, and the host layer
// keeps using the fp32-FMA kernel of core_gemm.cu.
#include "common.cuh"

namespace cagnet {

__device__ __forceinline__ float tf32_round(float x) {
  // nearest value with 10 explicit mantissa bits (ties away from zero; the remainder stays exact either way)
  return __int_as_float((__float_as_int(x) + 0x1000) & ~0x1fff);
}

__global__ void __launch_bounds__(256)
split_tf32_kernel(const float* __restrict__ x, int64_t count, float* __restrict__ hi, float* __restrict__ lo) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float v = x[i];
    const float h = tf32_round(v);
    hi[i] = h;
    lo[i] = v - h;
  }
}

// out[k, n] = hi(B[idx[k], n]), out[k, half + n] = lo(B[idx[k], n]) for n < f; columns [f, half) of both halves
// are written as zeros.  One thread per float4 of a gathered row.
__global__ void __launch_bounds__(256)
gather_split_rows_kernel(const float* __restrict__ B, int64_t ldb, const int* __restrict__ idx, int K, int f,
                         float* __restrict__ out, int64_t half) {
  const int vecs = static_cast<int>(half / 4);
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= static_cast<int64_t>(K) * vecs) return;
  const int k = static_cast<int>(t / vecs), n = static_cast<int>(t % vecs) * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (n < f) {
    const float4 q = __ldg(reinterpret_cast<const float4*>(B + static_cast<int64_t>(__ldg(idx + k)) * ldb + n));
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
  float h[4], l[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (n + j >= f) v[j] = 0.f;
    h[j] = tf32_round(v[j]);
    l[j] = v[j] - h[j];
  }
  float* row = out + static_cast<int64_t>(k) * 2 * half;
  *reinterpret_cast<float4*>(row + n) = make_float4(h[0], h[1], h[2], h[3]);
  *reinterpret_cast<float4*>(row + half + n) = make_float4(l[0], l[1], l[2], l[3]);
}

// C[rows[m], n] += D[m, n] + (D[m, half + n] + D[m, 2 half + n]): the hi*hi product plus the two cross products
// (small terms added to each other first).  One thread per float4.
__global__ void __launch_bounds__(256)
add_rows3_kernel(const float* __restrict__ D, int64_t half, const int* __restrict__ rows, int R,
                 float* __restrict__ C, int64_t ldc, int f) {
  const int vecs = static_cast<int>(half / 4);
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= static_cast<int64_t>(R) * vecs) return;
  const int m = static_cast<int>(t / vecs), n = static_cast<int>(t % vecs) * 4;
  if (n >= f) return;
  const float* d = D + static_cast<int64_t>(m) * 3 * half + n;
  const float4 a = __ldg(reinterpret_cast<const float4*>(d));
  const float4 b = __ldg(reinterpret_cast<const float4*>(d + half));
  const float4 c = __ldg(reinterpret_cast<const float4*>(d + 2 * half));
  float* out = C + static_cast<int64_t>(__ldg(rows + m)) * ldc + n;
  if (n + 0 < f) out[0] += a.x + (b.x + c.x);
  if (n + 1 < f) out[1] += a.y + (b.y + c.y);
  if (n + 2 < f) out[2] += a.z + (b.z + c.z);
  if (n + 3 < f) out[3] += a.w + (b.w + c.w);
}

static int g_core_chunk = 2048;
int core_chunk() { return g_core_chunk; }
int set_core_chunk(int value) {
  if (value < 256 || value % 32) return 1;
  g_core_chunk = value;
  return 0;
}

}  // namespace cagnet

#ifdef CAGNET_HAVE_CUTLASS

#include "cute/tensor.hpp"
#include "cutlass/cutlass.h"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/epilogue/thread/linear_combination.h"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/dispatch_policy.hpp"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/util/packed_stride.hpp"

namespace cagnet {
namespace tc {

using namespace cute;

using LayoutA = cutlass::layout::RowMajor;      // core: R x K, k contiguous
using LayoutB = cutlass::layout::RowMajor;      // [Bs_hi | Bs_lo]: K x N, n contiguous
using LayoutC = cutlass::layout::RowMajor;
constexpr int kAlign = 4;                       // 16-byte rows for TMA

using MmaTile = Shape<_128, _128, _32>;         // 128 x 256 tiles measured slower (1.24 against 1.02 ms at 13312^2)
using Cluster = Shape<_1, _1, _1>;

using Epilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, MmaTile, Cluster,
    cutlass::epilogue::collective::EpilogueTileAuto, float, float, float, LayoutC, kAlign, float, LayoutC, kAlign,
    cutlass::epilogue::collective::EpilogueScheduleAuto>::CollectiveOp;

// float operands on the tensor-op class = tcgen05.mma kind::tf32
using Mainloop = typename cutlass::gemm::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, float, LayoutA, kAlign, float, LayoutB, kAlign, float,
    MmaTile, Cluster,
    cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epilogue::SharedStorage))>,
    cutlass::gemm::collective::KernelScheduleAuto>::CollectiveOp;

using Kernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, Mainloop, Epilogue>;
using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;


static typename Gemm::Arguments make_args(const float* A, int64_t lda, const float* B, int64_t ldb, float* D,
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

// D (ldd) = beta * D + A (lda) * B (ldb) on `stream`
static int gemm(const float* A, int64_t lda, const float* B, int64_t ldb, float* D, int64_t ldd, int M, int N, int K,
                float beta, void* ws, size_t ws_bytes, cudaStream_t stream) {
  auto args = make_args(A, lda, B, ldb, D, ldd, M, N, K, beta);
  if (Gemm::get_workspace_size(args) > ws_bytes)
    return fail(CAGNET_E_WORKSPACE, "cagnet_core_gemm_tc_f32: workspace too small");
  Gemm op;
  if (op.can_implement(args) != cutlass::Status::kSuccess)
    return fail(CAGNET_E_ARG, "cagnet_core_gemm_tc_f32: shape or alignment not supported by the tensor-core mainloop");
  if (op.initialize(args, ws, stream) != cutlass::Status::kSuccess)
    return fail(CAGNET_E_LAUNCH, "cagnet_core_gemm_tc_f32: initialisation of the tensor-core multiply failed");
  if (op.run(stream) != cutlass::Status::kSuccess)
    return fail(CAGNET_E_LAUNCH, "cagnet_core_gemm_tc_f32: launch of the tensor-core multiply failed");
  return CAGNET_OK;
}

}  // namespace tc
}  // namespace cagnet

using namespace cagnet;

extern "C" int cagnet_core_gemm_tc_available(void) { return 1; }

extern "C" size_t cagnet_core_gemm_tc_workspace_bytes(int32_t R, int32_t K, int32_t f) {
  if (R <= 0 || K <= 0 || f <= 0) return 0;
  const int half = (f + 3) / 4 * 4;
  auto args = tc::make_args(nullptr, K, nullptr, 2 * half, nullptr, 3 * half, R, 2 * half, K < core_chunk() ? K : core_chunk(), 0.f);
  return tc::Gemm::get_workspace_size(args) + 16;
}

extern "C" int cagnet_core_gemm_tc_f32(const float* core_hi, const float* core_lo, int64_t ld_core, int32_t R, int32_t K,
                                       const float* Bs, int64_t half, float* D, int32_t f, void* ws, size_t ws_bytes,
                                       void* stream) {
  if (R < 0 || K < 0 || f < 0) return fail(CAGNET_E_ARG, "cagnet_core_gemm_tc_f32: negative size");
  if (R == 0 || K == 0 || f == 0) return CAGNET_OK;
  if (!core_hi || !core_lo || !Bs || !D) return fail(CAGNET_E_ARG, "cagnet_core_gemm_tc_f32: null pointer");
  if (ld_core < K || half < f) return fail(CAGNET_E_ARG, "cagnet_core_gemm_tc_f32: leading dimension too small");
  if (ld_core % 4 || half % 4 || !aligned(core_hi, 16) || !aligned(core_lo, 16) || !aligned(Bs, 16) || !aligned(D, 16))
    return fail(CAGNET_E_ALIGN, "cagnet_core_gemm_tc_f32: rows of the core, Bs and D must start on 16-byte boundaries");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int n1 = static_cast<int>(2 * half), n2 = static_cast<int>(half);
  const int chunk = core_chunk();
  for (int k0 = 0; k0 < K; k0 += chunk) {
    const int kc = (K - k0 < chunk) ? K - k0 : chunk;
    const float beta = k0 == 0 ? 0.f : 1.f;
    const float* b = Bs + static_cast<int64_t>(k0) * 2 * half;
    // D[:, 0:2 half) (+)= core_hi[:, k0:k0+kc) * [Bs_hi | Bs_lo][k0:k0+kc)
    int rc = tc::gemm(core_hi + k0, ld_core, b, 2 * half, D, 3 * half, R, n1, kc, beta, ws, ws_bytes, s);
    if (rc) return rc;
    // D[:, 2 half:3 half) (+)= core_lo[:, k0:k0+kc) * Bs_hi[k0:k0+kc)
    rc = tc::gemm(core_lo + k0, ld_core, b, 2 * half, D + 2 * half, 3 * half, R, n2, kc, beta, ws, ws_bytes, s);
    if (rc) return rc;
  }
  return check_launch("cagnet_core_gemm_tc_f32");
}

#else  // no CUTLASS header tree at build time

using namespace cagnet;

extern "C" int cagnet_core_gemm_tc_available(void) { return 0; }
extern "C" size_t cagnet_core_gemm_tc_workspace_bytes(int32_t, int32_t, int32_t) { return 0; }
extern "C" int cagnet_core_gemm_tc_f32(const float*, const float*, int64_t, int32_t, int32_t, const float*, int64_t,
                                       float*, int32_t, void*, size_t, void*) {
  return fail(CAGNET_E_ARG, "cagnet_core_gemm_tc_f32: built without the CUTLASS header tree");
}

#endif

extern "C" int cagnet_split_tf32_f32(const float* x, int64_t count, float* hi, float* lo, void* stream) {
  if (count < 0) return fail(CAGNET_E_ARG, "cagnet_split_tf32_f32: negative size");
  if (count == 0) return CAGNET_OK;
  if (!x || !hi || !lo) return fail(CAGNET_E_ARG, "cagnet_split_tf32_f32: null pointer");
  const int64_t blocks = (count + 255) / 256;
  split_tf32_kernel<<<static_cast<unsigned>(blocks < 16 * kNumSMs ? blocks : 16 * kNumSMs), 256, 0,
                      static_cast<cudaStream_t>(stream)>>>(x, count, hi, lo);
  return check_launch("cagnet_split_tf32_f32");
}

extern "C" int cagnet_gather_split_rows_f32(const float* B, int64_t ldb, const int32_t* idx, int32_t K, int32_t f,
                                            float* out, int64_t half, void* stream) {
  if (K < 0 || f < 0) return fail(CAGNET_E_ARG, "cagnet_gather_split_rows_f32: negative size");
  if (K == 0 || f == 0) return CAGNET_OK;
  if (!B || !idx || !out) return fail(CAGNET_E_ARG, "cagnet_gather_split_rows_f32: null pointer");
  const int64_t f4 = (static_cast<int64_t>(f) + 3) / 4 * 4;
  if (ldb < f4 || half < f4 || ldb % 4 || half % 4 || !aligned(B, 16) || !aligned(out, 16))
    return fail(CAGNET_E_ALIGN, "cagnet_gather_split_rows_f32: rows must be padded to a multiple of 4 floats and 16-byte aligned");
  const int64_t threads = static_cast<int64_t>(K) * (half / 4);
  gather_split_rows_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      B, ldb, idx, K, f, out, half);
  return check_launch("cagnet_gather_split_rows_f32");
}

extern "C" int cagnet_add_rows3_f32(const float* D, int64_t half, const int32_t* rows, int32_t R, int32_t f, float* C,
                                    int64_t ldc, void* stream) {
  if (R < 0 || f < 0) return fail(CAGNET_E_ARG, "cagnet_add_rows3_f32: negative size");
  if (R == 0 || f == 0) return CAGNET_OK;
  if (!D || !rows || !C) return fail(CAGNET_E_ARG, "cagnet_add_rows3_f32: null pointer");
  if (half < f || ldc < f || half % 4 || !aligned(D, 16))
    return fail(CAGNET_E_ALIGN, "cagnet_add_rows3_f32: D rows must be padded to a multiple of 4 floats and 16-byte aligned");
  const int64_t threads = static_cast<int64_t>(R) * (half / 4);
  add_rows3_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      D, half, rows, R, C, ldc, f);
  return check_launch("cagnet_add_rows3_f32");
}
