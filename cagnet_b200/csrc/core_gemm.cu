// Dense core of a power-law adjacency block for sm_100a.
//
// In a scale-free graph the hub rows meet the hub columns in a sub-block that is far from sparse: on the
// 233K-vertex / 115M-nonzero R-MAT benchmark graph the 8192 x 8192 block of the highest-degree rows and columns
// holds 26 M nonzeros (39 % dense, 23 % of the matrix).  Gathering a 2.4 KB row of B per nonzero costs more there
// than multiplying the block as a dense matrix, because a dense tile re-uses every row of B it stages in shared
// memory 128 times.  The host layer cuts that core out of the CSR block once; per multiply it calls
//
//     C[rows[i], :] += sum_j core[i, j] * B[cols[j], :]          i < R, j < K
//
// which is an fp32 SGEMM whose B rows and C rows are addressed through the two index lists (no gathered copy of
// B, no scatter pass).  128 x 128 output tiles, 256 threads, 8 x 8 accumulators per thread, 16-deep k steps,
// the next step's operands fetched into registers while the current one is multiplied.  Plain fp32 FMAs in a
// fixed order: deterministic, and as accurate as the sparse kernel it replaces.
//
// The core has few rows (thousands) and few column tiles (five at width 602), so its output tiles alone cannot
// fill 148 SMs evenly: 160 tiles on 296 resident blocks ran at 22 TFLOP/s.  The k range is therefore cut into
// `parts` slices, one block per (tile, slice); the slices write partial tiles to a workspace and a second kernel
// adds them up in slice order into the listed rows of C.  The partial tiles are tiny next to the multiply
// (R x f x parts floats), and the order of additions is fixed, so the result is still reproducible.
#include "common.cuh"

namespace cagnet {

constexpr int kCoreBM = 128, kCoreBN = 128, kCoreBK = 16;
constexpr int kCorePadM = kCoreBM + 4;      // row pitch of the transposed A tile (store-side bank spread)

__global__ void __launch_bounds__(256, 2)
core_gemm_kernel(const float* __restrict__ core, int64_t ld_core, const int* __restrict__ rows, int R,
                 const int* __restrict__ cols, int K, const float* __restrict__ B, int64_t ldb,
                 float* __restrict__ C, int64_t ldc, int f, int k_per_part, float* __restrict__ ws, int64_t ldw) {
  __shared__ __align__(16) float As[2][kCoreBK][kCorePadM];   // As[k][m] = core[m0 + m][k0 + k]
  __shared__ __align__(16) float Bs[2][kCoreBK][kCoreBN];     // Bs[k][n] = B[cols[k0 + k]][n0 + n]
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * kCoreBN;
  const int m0 = blockIdx.y * kCoreBM;
  const int tx = tid & 15, ty = tid >> 4;

  // loader roles: A tile 128 x 16 = 512 float4 (two per thread, along k); B tile 16 x 128 = 512 float4
  const int a_row = tid >> 2;            // 0..63 (+64)
  const int a_k = (tid & 3) * 4;         // 0,4,8,12
  const int b_k = tid >> 5;              // 0..7 (+8)
  const int b_col = (tid & 31) * 4;      // 0..124
  const bool core_vec4 = (ld_core % 4 == 0) && aligned(core, 16);
  // columns of B that may be read as a whole float4: inside the allocated row (pad columns hold anything;
  // their products are never stored)
  const bool b_ok = (n0 + b_col + 3) < ldb && (n0 + b_col) < ((f + 3) / 4 * 4);

  float4 a_reg[2], b_reg[2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int m = m0 + a_row + 64 * h;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m < R) {
        const float* p = core + static_cast<int64_t>(m) * ld_core + k0 + a_k;
        if (core_vec4 && k0 + a_k + 3 < K) {
          v = __ldg(reinterpret_cast<const float4*>(p));
        } else {
          if (k0 + a_k + 0 < K) v.x = __ldg(p + 0);
          if (k0 + a_k + 1 < K) v.y = __ldg(p + 1);
          if (k0 + a_k + 2 < K) v.z = __ldg(p + 2);
          if (k0 + a_k + 3 < K) v.w = __ldg(p + 3);
        }
      }
      a_reg[h] = v;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int k = k0 + b_k + 8 * h;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k < K && b_ok) {
        const int r = __ldg(cols + k);
        v = __ldg(reinterpret_cast<const float4*>(B + static_cast<int64_t>(r) * ldb + n0 + b_col));
      }
      b_reg[h] = v;
    }
  };
  auto park = [&](int buf) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int m = a_row + 64 * h;
      As[buf][a_k + 0][m] = a_reg[h].x;
      As[buf][a_k + 1][m] = a_reg[h].y;
      As[buf][a_k + 2][m] = a_reg[h].z;
      As[buf][a_k + 3][m] = a_reg[h].w;
      *reinterpret_cast<float4*>(&Bs[buf][b_k + 8 * h][b_col]) = b_reg[h];
    }
  };

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  const int k_begin = blockIdx.z * k_per_part;        // k_per_part is a multiple of the k step
  K = min(K, k_begin + k_per_part);                   // the loaders zero-fill beyond this slice's end
  const int steps = (K - k_begin + kCoreBK - 1) / kCoreBK;
  fetch(k_begin);
  park(0);
  __syncthreads();
  for (int s = 0; s < steps; ++s) {
    const int cur = s & 1;
    if (s + 1 < steps) fetch(k_begin + (s + 1) * kCoreBK);
#pragma unroll
    for (int k = 0; k < kCoreBK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[cur][k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[cur][k][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[cur][k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[cur][k][64 + tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (s + 1 < steps) park(cur ^ 1);    // the other buffer was last read before the previous barrier
    __syncthreads();
  }

  if (ws) {
    // partial tile of this k slice: ws[slice][m][n], rows padded to ldw (a multiple of 4, 16-byte aligned base)
    float* part = ws + static_cast<int64_t>(blockIdx.z) * R * ldw;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
      if (m >= R) continue;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int n = n0 + 64 * h + tx * 4;
        if (n < ldw)
          *reinterpret_cast<float4*>(part + static_cast<int64_t>(m) * ldw + n) =
              make_float4(acc[i][4 * h + 0], acc[i][4 * h + 1], acc[i][4 * h + 2], acc[i][4 * h + 3]);
      }
    }
    return;
  }
  // C rows are reached through the row list; every listed row is distinct, so plain read-modify-write
  const bool c_vec4 = (ldc % 4 == 0) && aligned(C, 16);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (m >= R) continue;
    float* crow = C + static_cast<int64_t>(__ldg(rows + m)) * ldc;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = n0 + 64 * h + tx * 4;
      if (c_vec4 && n + 3 < f) {
        float4 v = *reinterpret_cast<float4*>(crow + n);
        v.x += acc[i][4 * h + 0]; v.y += acc[i][4 * h + 1]; v.z += acc[i][4 * h + 2]; v.w += acc[i][4 * h + 3];
        *reinterpret_cast<float4*>(crow + n) = v;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n + j < f) crow[n + j] += acc[i][4 * h + j];
      }
    }
  }
}

// C[rows[m], n] += ws[0][m][n] + ws[1][m][n] + ... in slice order.  One thread per float4 of a core row.
__global__ void __launch_bounds__(256)
core_reduce_kernel(const float* __restrict__ ws, int64_t ldw, int parts, const int* __restrict__ rows, int R,
                   float* __restrict__ C, int64_t ldc, int f) {
  const int vecs = static_cast<int>(ldw / 4);
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= static_cast<int64_t>(R) * vecs) return;
  const int m = static_cast<int>(t / vecs), n = static_cast<int>(t % vecs) * 4;
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int p = 0; p < parts; ++p) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(ws + (static_cast<int64_t>(p) * R + m) * ldw + n));
    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
  }
  float* c = C + static_cast<int64_t>(__ldg(rows + m)) * ldc + n;
  if (n + 0 < f) c[0] += sum.x;
  if (n + 1 < f) c[1] += sum.y;
  if (n + 2 < f) c[2] += sum.z;
  if (n + 3 < f) c[3] += sum.w;
}

// How many k slices: enough blocks for about six full waves of 2 blocks per SM, so that the last wave's idle SMs
// cost little, but never slices shorter than 16 k steps.
static int core_parts(int R, int K, int f) {
  const int64_t tiles = static_cast<int64_t>((f + kCoreBN - 1) / kCoreBN) * ((R + kCoreBM - 1) / kCoreBM);
  const int64_t target = 6LL * 2 * kNumSMs;
  int64_t parts = (target + tiles - 1) / tiles;
  const int64_t longest = (K + 16 * kCoreBK - 1) / (16 * kCoreBK);
  if (parts > longest) parts = longest;
  if (parts < 1) parts = 1;
  return static_cast<int>(parts);
}

static int64_t core_ldw(int f) { return (static_cast<int64_t>(f) + 3) / 4 * 4; }

}  // namespace cagnet

using namespace cagnet;

extern "C" size_t cagnet_core_gemm_workspace_bytes(int32_t R, int32_t K, int32_t f) {
  if (R <= 0 || K <= 0 || f <= 0) return 0;
  const int parts = core_parts(R, K, f);
  return parts <= 1 ? 0 : static_cast<size_t>(parts) * R * core_ldw(f) * sizeof(float);
}

extern "C" int cagnet_core_gemm_f32(const float* core, int64_t ld_core, const int32_t* core_rows, int32_t R,
                                    const int32_t* core_cols, int32_t K, const float* B, int64_t ldb, float* C,
                                    int64_t ldc, int32_t f, void* ws, size_t ws_bytes, void* stream) {
  if (R < 0 || K < 0 || f < 0) return fail(CAGNET_E_ARG, "cagnet_core_gemm_f32: negative size");
  if (R == 0 || K == 0 || f == 0) return CAGNET_OK;
  if (!core || !core_rows || !core_cols || !B || !C) return fail(CAGNET_E_ARG, "cagnet_core_gemm_f32: null pointer");
  if (ld_core < K || ldb < f || ldc < f) return fail(CAGNET_E_ARG, "cagnet_core_gemm_f32: leading dimension too small");
  if (ldb % 4 != 0 || !aligned(B, 16))
    return fail(CAGNET_E_ALIGN, "cagnet_core_gemm_f32: B rows must start on 16-byte boundaries (ldb %% 4 == 0)");
  const int parts = core_parts(R, K, f);
  const size_t need = cagnet_core_gemm_workspace_bytes(R, K, f);
  if (need && (!ws || ws_bytes < need || !aligned(ws, 16)))
    return fail(CAGNET_E_WORKSPACE, "cagnet_core_gemm_f32: workspace of %s%lld bytes is too small or misaligned (need %lld)",
                "", (long long)ws_bytes, (long long)need);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int k_per_part = (K + parts - 1) / parts;
  k_per_part = (k_per_part + kCoreBK - 1) / kCoreBK * kCoreBK;
  const int64_t ldw = core_ldw(f);
  const dim3 grid((f + kCoreBN - 1) / kCoreBN, (R + kCoreBM - 1) / kCoreBM, parts);
  core_gemm_kernel<<<grid, 256, 0, s>>>(core, ld_core, core_rows, R, core_cols, K, B, ldb, C, ldc, f, k_per_part,
                                        parts > 1 ? static_cast<float*>(ws) : nullptr, ldw);
  if (parts > 1) {
    const int64_t threads = static_cast<int64_t>(R) * (ldw / 4);
    core_reduce_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, s>>>(static_cast<const float*>(ws), ldw,
                                                                                   parts, core_rows, R, C, ldc, f);
  }
  return check_launch("cagnet_core_gemm_f32");
}
