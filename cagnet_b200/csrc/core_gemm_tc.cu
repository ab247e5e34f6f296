// Dense core of a power-law adjacency block on the 5th-generation tensor cores (tcgen05 / TMEM) of sm_100a.
//
// D[R x f] = core[R x K] * Bs[K x f], all fp32 in memory.  The multiply runs as CUTLASS's sm100 "fast FP32"
// mainloop: TMA brings fp32 tiles of both operands into shared memory, transform warps split every value into
// three bf16 terms (x = x1 + 2^-8 x2 + 2^-16 x3; the terms of A go to TMEM, those of B back to shared memory),
// tcgen05.mma accumulates the cross products into TMEM, and the accumulator is promoted to fp32 registers after
// every k block, so that the result carries fp32 accuracy (not TF32's 10 bits) while the contraction itself runs
// on the tensor pipe.  Of the nine cross products the three of order 2^-24 and below are left out (the builder's
// default computes all nine; measured 2.66 ms against 2.74 ms at 16384^2 x 608, the same 1.3e-6 error against
// fp64).  One CTA per 128 x 128 output tile, cluster shape 1 x 1 x 1 (every CTA loads its own tiles), 1-SM MMA.
// Measured: 123 TFLOP/s fp32-equivalent at 16384 x 16384 x 608, against 40 for the fp32-FMA kernel of
// core_gemm.cu and 47-57 for the library SGEMM.
//
// This file only instantiates the CUTLASS / CuTe templates (header tree found at build time); the gather of B's
// rows before it and the addition of D into C's rows after it are kernels of this library (core_gemm.cu).
// Without the header tree the file compiles to a stub that reports CAGNET_E_ARG, and the host layer keeps using
// the fp32-FMA kernel.
#include "common.cuh"

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

using ElementA = float;                         // core, row-major R x K  (K contiguous)
using ElementB = float;                         // Bs, row-major K x f    (f contiguous: "row-major B")
using ElementC = float;
using ElementAcc = float;
using LayoutA = cutlass::layout::RowMajor;
using LayoutB = cutlass::layout::RowMajor;
using LayoutC = cutlass::layout::RowMajor;
constexpr int kAlign = 4;                       // 16-byte rows for TMA

using MmaTile = Shape<_128, _128, _32>;
using Cluster = Shape<_1, _1, _1>;

using Epilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, MmaTile, Cluster,
    cutlass::epilogue::collective::EpilogueTileAuto, ElementAcc, ElementAcc, ElementC, LayoutC, kAlign, ElementC,
    LayoutC, kAlign, cutlass::epilogue::FastF32NoSmemWarpSpecialized1Sm>::CollectiveOp;

using Built = typename cutlass::gemm::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, ElementA, LayoutA, kAlign, ElementB, LayoutB, kAlign,
    ElementAcc, MmaTile, Cluster,
    cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epilogue::SharedStorage))>,
    cutlass::gemm::KernelTmaWarpSpecialized1SmFastFP32Sm100>::CollectiveOp;

// the builder's mainloop with one change: 3 bands (6 cross products) instead of 5 (9)
constexpr int kBands = 3;
using BuiltPolicy = typename Built::DispatchPolicy;
using Policy = cutlass::gemm::MainloopSm100TmaUmmaWarpSpecializedFastF32<
    BuiltPolicy::Load2TransformPipelineStageCount, BuiltPolicy::Transform2MmaPipelineStageCount,
    BuiltPolicy::Schedule::SchedulerPipelineStageCount, BuiltPolicy::Schedule::AccumulatorPipelineStageCount, kBands,
    BuiltPolicy::ScalingFactor, BuiltPolicy::AccPromotionInterval, typename BuiltPolicy::ClusterShape,
    typename BuiltPolicy::AccumulatorCopyAtom, typename BuiltPolicy::ArchTag>;
using Mainloop = cutlass::gemm::collective::CollectiveMma<
    Policy, typename Built::TileShape, float, typename Built::StrideA, float, typename Built::StrideB,
    typename Built::TiledMma, typename Built::GmemTiledCopyA, typename Built::SmemLayoutAtomsA,
    typename Built::CopyAtomsA, typename Built::TransformA, typename Built::GmemTiledCopyB,
    typename Built::SmemLayoutAtomsB, typename Built::CopyAtomsB, typename Built::TransformB>;

using Kernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, Mainloop, Epilogue>;
using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;

static typename Gemm::Arguments make_args(const float* core, int64_t ld_core, int R, int K, const float* Bs, int64_t ldbs,
                                          float* D, int64_t ldd, int f) {
  using StrideA = typename Kernel::StrideA;
  using StrideB = typename Kernel::StrideB;
  using StrideC = typename Kernel::StrideC;
  using StrideD = typename Kernel::StrideD;
  StrideA sa = cutlass::make_cute_packed_stride(StrideA{}, cute::make_shape(R, K, 1));
  StrideB sb = cutlass::make_cute_packed_stride(StrideB{}, cute::make_shape(f, K, 1));
  StrideC sc = cutlass::make_cute_packed_stride(StrideC{}, cute::make_shape(R, f, 1));
  StrideD sd = cutlass::make_cute_packed_stride(StrideD{}, cute::make_shape(R, f, 1));
  // leading dimensions of the padded layouts (the packed helpers assume ld == extent)
  cute::get<0>(sa) = ld_core;
  cute::get<1>(sb) = ldbs;
  cute::get<0>(sc) = ldd;
  cute::get<0>(sd) = ldd;
  typename Gemm::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm,
                                {R, f, K, 1},
                                {core, sa, Bs, sb},
                                {{1.0f, 0.0f}, D, sc, D, sd}};
  return args;
}

}  // namespace tc
}  // namespace cagnet

using namespace cagnet;

extern "C" int cagnet_core_gemm_tc_available(void) { return 1; }

extern "C" size_t cagnet_core_gemm_tc_workspace_bytes(int32_t R, int32_t K, int32_t f) {
  if (R <= 0 || K <= 0 || f <= 0) return 0;
  const int f4 = (f + 3) / 4 * 4;
  auto args = tc::make_args(nullptr, K, R, K, nullptr, f4, nullptr, f4, f4);
  return tc::Gemm::get_workspace_size(args) + 16;
}

extern "C" int cagnet_core_gemm_tc_f32(const float* core, int64_t ld_core, int32_t R, int32_t K, const float* Bs,
                                       int64_t ldbs, float* D, int64_t ldd, int32_t f, void* ws, size_t ws_bytes,
                                       void* stream) {
  if (R < 0 || K < 0 || f < 0) return fail(CAGNET_E_ARG, "cagnet_core_gemm_tc_f32: negative size");
  if (R == 0 || K == 0 || f == 0) return CAGNET_OK;
  if (!core || !Bs || !D) return fail(CAGNET_E_ARG, "cagnet_core_gemm_tc_f32: null pointer");
  if (ld_core < K || ldbs < f || ldd < f) return fail(CAGNET_E_ARG, "cagnet_core_gemm_tc_f32: leading dimension too small");
  if (ld_core % 4 || ldbs % 4 || ldd % 4 || !aligned(core, 16) || !aligned(Bs, 16) || !aligned(D, 16))
    return fail(CAGNET_E_ALIGN, "cagnet_core_gemm_tc_f32: rows of core, Bs and D must start on 16-byte boundaries");
  // the mainloop wants whole 16-byte vectors along f: columns [f, f4) are pad columns of Bs and D (their values
  // are unspecified on the way in and on the way out; no other column depends on them)
  const int f4 = (f + 3) / 4 * 4;
  if (ldbs < f4 || ldd < f4) return fail(CAGNET_E_ARG, "cagnet_core_gemm_tc_f32: rows must be padded to a multiple of 4 floats");
  auto args = tc::make_args(core, ld_core, R, K, Bs, ldbs, D, ldd, f4);
  const size_t need = tc::Gemm::get_workspace_size(args);
  if (need && (!ws || ws_bytes < need))
    return fail(CAGNET_E_WORKSPACE, "cagnet_core_gemm_tc_f32: workspace of %s%lld bytes is too small (need %lld)", "",
                (long long)ws_bytes, (long long)need);
  tc::Gemm gemm;
  if (gemm.can_implement(args) != cutlass::Status::kSuccess)
    return fail(CAGNET_E_ARG, "cagnet_core_gemm_tc_f32: shape or alignment not supported by the tensor-core mainloop");
  if (gemm.initialize(args, ws, static_cast<cudaStream_t>(stream)) != cutlass::Status::kSuccess)
    return fail(CAGNET_E_LAUNCH, "cagnet_core_gemm_tc_f32: initialisation of the tensor-core multiply failed");
  if (gemm.run(static_cast<cudaStream_t>(stream)) != cutlass::Status::kSuccess)
    return fail(CAGNET_E_LAUNCH, "cagnet_core_gemm_tc_f32: launch of the tensor-core multiply failed");
  return check_launch("cagnet_core_gemm_tc_f32");
}

#else  // no CUTLASS header tree at build time

using namespace cagnet;

extern "C" int cagnet_core_gemm_tc_available(void) { return 0; }
extern "C" size_t cagnet_core_gemm_tc_workspace_bytes(int32_t, int32_t, int32_t) { return 0; }
extern "C" int cagnet_core_gemm_tc_f32(const float*, int64_t, int32_t, int32_t, const float*, int64_t, float*, int64_t,
                                       int32_t, void*, size_t, void*) {
  return fail(CAGNET_E_ARG, "cagnet_core_gemm_tc_f32: built without the CUTLASS header tree");
}

#endif
