// Dense side of the GCN layer for sm_100a: tall-skinny fp32 products with fused activations,
// the split-row weight-gradient product, row-wise log-softmax and the masked NLL loss.
//
// All of these are HBM-bound at GCN shapes (a 233K x 602 operand against a 602 x 16 weight has
// ~7 flop/byte), so they run on the fp32 FMA pipes from shared-memory tiles: the tall operand is
// read exactly once, coalesced; the small operand lives in shared memory.
#include <limits.h>
#include <math.h>

#include "common.cuh"

namespace cagnet {

// ------------------------------------------------------------------------------------------------
// Z[n x N] = epilogue(X[n x K] * W)       block: 128 rows x (8*TN) columns, 256 threads
// thread (rg = tid/8, cg = tid%8) owns rows rg*4..rg*4+3 and columns cg + 8*t, t < TN.
constexpr int kBM = 128;
constexpr int kBK = 32;

template <int TN>
__global__ void __launch_bounds__(256) gemm_nn_kernel(const float* __restrict__ X, int64_t ldx,
                                                      const float* __restrict__ W, int64_t ldw, int transW,
                                                      float* __restrict__ Z, int64_t ldz, int64_t n, int K, int N,
                                                      int epilogue, const float* __restrict__ aux, int64_t ldaux,
                                                      int x_vec4) {
  constexpr int NT = 8 * TN;
  __shared__ float Xs[kBK][kBM + 1];
  __shared__ float Ws[kBK][NT];
  const int tid = threadIdx.x;
  const int cg = tid & 7, rg = tid >> 3;
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * kBM;
  const int n0 = blockIdx.y * NT;

  float acc[4][TN];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int t = 0; t < TN; ++t) acc[i][t] = 0.f;

  // The X tile of step k+1 is fetched into registers while step k is being multiplied, so the kernel waits for
  // HBM once per tile instead of once per tile and synchronisation.
  constexpr int WPT = (kBK * NT + 255) / 256;     // W elements per thread and step
  const int kk = (tid & 7) * 4;
  float xv[4][4];
  float wv[WPT];

  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t gr = row0 + (tid >> 3) + 32 * i;
#pragma unroll
      for (int j = 0; j < 4; ++j) xv[i][j] = 0.f;
      if (gr < n) {
        const float* xp = X + gr * ldx + k0 + kk;
        if (x_vec4 && k0 + kk + 3 < K) {
          const float4 t4 = __ldg(reinterpret_cast<const float4*>(xp));
          xv[i][0] = t4.x; xv[i][1] = t4.y; xv[i][2] = t4.z; xv[i][3] = t4.w;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (k0 + kk + j < K) xv[i][j] = __ldg(xp + j);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < WPT; ++u) {
      const int idx = tid + 256 * u;
      const int k = idx / NT, j = idx % NT;
      float w = 0.f;
      if (idx < kBK * NT && k0 + k < K && n0 + j < N)
        w = transW ? __ldg(W + static_cast<int64_t>(n0 + j) * ldw + k0 + k) : __ldg(W + static_cast<int64_t>(k0 + k) * ldw + n0 + j);
      wv[u] = w;
    }
  };

  fetch(0);
  for (int k0 = 0; k0 < K; k0 += kBK) {
    // X tile: 128 rows x 32 k, read row-contiguous, stored k-major; W tile: 32 k x NT columns
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) Xs[kk + j][(tid >> 3) + 32 * i] = xv[i][j];
#pragma unroll
    for (int u = 0; u < WPT; ++u) {
      const int idx = tid + 256 * u;
      if (idx < kBK * NT) Ws[idx / NT][idx % NT] = wv[u];
    }
    __syncthreads();
    if (k0 + kBK < K) fetch(k0 + kBK);
#pragma unroll 8
    for (int k = 0; k < kBK; ++k) {
      float x[4], w[TN];
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = Xs[k][rg * 4 + i];
#pragma unroll
      for (int t = 0; t < TN; ++t) w[t] = Ws[k][cg + 8 * t];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int t = 0; t < TN; ++t) acc[i][t] = fmaf(x[i], w[t], acc[i][t]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gr = row0 + rg * 4 + i;
    const bool row_ok = gr < n;   // no early exit: the shuffles below need all 32 lanes
    if (epilogue == CAGNET_EPI_LOG_SOFTMAX) {
      float mx = -INFINITY;
#pragma unroll
      for (int t = 0; t < TN; ++t)
        if (n0 + cg + 8 * t < N) mx = fmaxf(mx, acc[i][t]);
#pragma unroll
      for (int off = 1; off < 8; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      float sum = 0.f;
#pragma unroll
      for (int t = 0; t < TN; ++t)
        if (n0 + cg + 8 * t < N) sum += expf(acc[i][t] - mx);
#pragma unroll
      for (int off = 1; off < 8; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      const float lse = mx + logf(sum);
#pragma unroll
      for (int t = 0; t < TN; ++t) acc[i][t] -= lse;
    }
    if (!row_ok) continue;
#pragma unroll
    for (int t = 0; t < TN; ++t) {
      const int c = n0 + cg + 8 * t;
      if (c < N) {
        float v = acc[i][t];
        if (epilogue == CAGNET_EPI_RELU) v = fmaxf(v, 0.f);
        else if (epilogue == CAGNET_EPI_RELU_MASK) v = (__ldg(aux + gr * ldaux + c) > 0.f) ? v : 0.f;
        else if (epilogue == CAGNET_EPI_ACCUMULATE) v += Z[gr * ldz + c];
        Z[gr * ldz + c] = v;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// out[K x N] = H^T * G over n rows.  grid (chunks, K tiles of 64, N tiles of 64).  Each block
// streams its row chunk 32 rows at a time through shared memory and keeps a 64 x NT tile of
// partial sums in registers: unit u = (k = u % 64, 4 columns jb = u / 64).
constexpr int kTnKT = 64;
constexpr int kTnNT = 64;
constexpr int kTnRB = 32;

__global__ void __launch_bounds__(256) gemm_tn_partial_kernel(const float* __restrict__ H, int64_t ldh,
                                                              const float* __restrict__ G, int64_t ldg, int64_t n,
                                                              int K, int N, int64_t rows_per_chunk,
                                                              float* __restrict__ ws) {
  __shared__ float Hs[kTnRB][kTnKT];
  __shared__ __align__(16) float Gs[kTnRB][kTnNT];
  const int tid = threadIdx.x;
  const int k0 = blockIdx.y * kTnKT, n0 = blockIdx.z * kTnNT;
  const int64_t r_begin = static_cast<int64_t>(blockIdx.x) * rows_per_chunk;
  const int64_t r_end = min(n, r_begin + rows_per_chunk);
  const int nt = min(kTnNT, N - n0);        // live columns of this tile
  const int nb = (nt + 3) / 4;              // 4-column groups
  const int units = kTnKT * nb;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // 32 rows of H (64 columns) and G (up to 64 columns) per step: 8 + 8 values per thread, fetched into registers
  // one step ahead of the multiply.
  float hv[8], gv[8];
  auto fetch = [&](int64_t r0) {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int idx = tid + 256 * u;
      const int r = idx / kTnKT, k = idx % kTnKT;
      hv[u] = (r0 + r < r_end && k0 + k < K) ? __ldg(H + (r0 + r) * ldh + k0 + k) : 0.f;
      const int j = idx % kTnNT;
      gv[u] = (r0 + r < r_end && j < nt) ? __ldg(G + (r0 + r) * ldg + n0 + j) : 0.f;
    }
  };
  if (r_begin < r_end) fetch(r_begin);
  for (int64_t r0 = r_begin; r0 < r_end; r0 += kTnRB) {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int idx = tid + 256 * u;
      Hs[idx / kTnKT][idx % kTnKT] = hv[u];
      Gs[idx / kTnNT][idx % kTnNT] = gv[u];
    }
    __syncthreads();
    if (r0 + kTnRB < r_end) fetch(r0 + kTnRB);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int u = tid + 256 * i;
      if (u < units) {
        const int k = u % kTnKT, jb = u / kTnKT;
#pragma unroll 8
        for (int r = 0; r < kTnRB; ++r) {
          const float h = Hs[r][k];
          const float4 g = *reinterpret_cast<const float4*>(&Gs[r][jb * 4]);
          acc[i][0] = fmaf(h, g.x, acc[i][0]);
          acc[i][1] = fmaf(h, g.y, acc[i][1]);
          acc[i][2] = fmaf(h, g.z, acc[i][2]);
          acc[i][3] = fmaf(h, g.w, acc[i][3]);
        }
      }
    }
    __syncthreads();
  }
  float* wp = ws + static_cast<int64_t>(blockIdx.x) * K * N;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int u = tid + 256 * i;
    if (u < units) {
      const int k = k0 + u % kTnKT, jb = u / kTnKT;
      if (k < K) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = n0 + jb * 4 + j;
          if (c < N) wp[static_cast<int64_t>(k) * N + c] = acc[i][j];
        }
      }
    }
  }
}

// The same product for N <= 16 (the weight gradients of the 602 x 16 layer: H is the 233K x 602 feature matrix,
// G has 16 columns).  There the kernel above spends two shared-memory reads on four FMAs, prefetches one step
// ahead and runs at 1.4 TB/s of H with its warps waiting on the loads.  Here
//   * a thread owns 4 consecutive k and all 16 columns (64 accumulators) for one sixteenth of the rows of a step:
//     one 128-bit read of H and four of G feed 64 FMAs;
//   * the tiles of the next three steps are already on their way: 16-byte cp.async copies into a four-stage ring
//     of shared-memory tiles (64 rows x 64 columns of H and 64 x 16 of G per stage), out-of-range rows and
//     columns zero-filled by the copy's source size.
// Threads that share their k columns (same tid % 16) are summed at the end, first by a shuffle inside each warp,
// then over the 8 warps in warp order.  Needs 16-byte aligned rows of H and G.
constexpr int kTnSmallRB = 64;       // rows per step
constexpr int kTnSmallStages = 4;
constexpr int kTnSmallStageFloats = kTnSmallRB * kTnKT + kTnSmallRB * 16;
constexpr int kTnSmallSmemBytes = kTnSmallStages * kTnSmallStageFloats * 4;     // 80 KB; also holds the 32 KB of sums

__device__ __forceinline__ void cp_async16(float* smem_dst, const float* gmem_src, int src_bytes) {
  const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem_src), "r"(src_bytes) : "memory");
}

__global__ void __launch_bounds__(256, 2) gemm_tn_small_kernel(const float* __restrict__ H, int64_t ldh,
                                                               const float* __restrict__ G, int64_t ldg, int64_t n,
                                                               int K, int N, int64_t rows_per_chunk,
                                                               float* __restrict__ ws) {
  extern __shared__ __align__(16) float tn_smem[];
  const int tid = threadIdx.x;
  const int kq = tid & 15, rs = tid >> 4;
  const int k0 = blockIdx.y * kTnKT;
  const int64_t r_begin = static_cast<int64_t>(blockIdx.x) * rows_per_chunk;
  const int64_t r_end = min(n, r_begin + rows_per_chunk);
  const int steps = static_cast<int>((r_end - r_begin + kTnSmallRB - 1) / kTnSmallRB);

  // copies of one step: 4 float4 of H and 1 float4 of G per thread
  auto issue = [&](int step) {
    if (step < steps) {
      float* hs = tn_smem + (step % kTnSmallStages) * kTnSmallStageFloats;
      float* gs = hs + kTnSmallRB * kTnKT;
      const int64_t r0 = r_begin + static_cast<int64_t>(step) * kTnSmallRB;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = tid + 256 * u;             // float4 index in the H tile
        const int r = idx >> 4, c = (idx & 15) * 4;
        const int k = k0 + c;
        int bytes = (r0 + r < r_end) ? (K - k) * 4 : 0;
        bytes = bytes < 0 ? 0 : (bytes > 16 ? 16 : bytes);
        const float* src = bytes ? H + (r0 + r) * ldh + k : H;
        cp_async16(hs + r * kTnKT + c, src, bytes);
      }
      const int r = tid >> 2, j = (tid & 3) * 4;
      int bytes = (r0 + r < r_end) ? (N - j) * 4 : 0;
      bytes = bytes < 0 ? 0 : (bytes > 16 ? 16 : bytes);
      const float* src = bytes ? G + (r0 + r) * ldg + j : G;
      cp_async16(gs + r * 16 + j, src, bytes);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");     // an empty group keeps the count in step
  };

  float acc[4][16];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[i][j] = 0.f;

#pragma unroll
  for (int s = 0; s < kTnSmallStages - 1; ++s) issue(s);
  for (int step = 0; step < steps; ++step) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kTnSmallStages - 2) : "memory");   // this step's tiles have landed
    __syncthreads();                     // ... for every thread, and everyone is done with the stage refilled next
    issue(step + kTnSmallStages - 1);
    const float* hs = tn_smem + (step % kTnSmallStages) * kTnSmallStageFloats;
    const float* gs = hs + kTnSmallRB * kTnKT;
#pragma unroll
    for (int q = 0; q < kTnSmallRB / 16; ++q) {
      const int r = rs + 16 * q;
      const float4 h4 = *reinterpret_cast<const float4*>(hs + r * kTnKT + kq * 4);
      const float h[4] = {h4.x, h4.y, h4.z, h4.w};
      float g[16];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float4 g4 = *reinterpret_cast<const float4*>(gs + r * 16 + c * 4);
        g[4 * c + 0] = g4.x; g[4 * c + 1] = g4.y; g[4 * c + 2] = g4.z; g[4 * c + 3] = g4.w;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[i][j] = fmaf(h[i], g[j], acc[i][j]);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();                       // the ring is free: it now holds the partial sums of the 8 warps
  float (*red)[16][64] = reinterpret_cast<float (*)[16][64]>(tn_smem);
  // lanes l and l + 16 of a warp hold the same k columns for two row subsets
  const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[i][j] += __shfl_down_sync(0xffffffffu, acc[i][j], 16);
  if (lane < 16) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 16; j += 4)
        *reinterpret_cast<float4*>(&red[warp][lane][i * 16 + j]) =
            make_float4(acc[i][j], acc[i][j + 1], acc[i][j + 2], acc[i][j + 3]);
  }
  __syncthreads();
  float* wp = ws + static_cast<int64_t>(blockIdx.x) * K * N;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int e = tid + 256 * u;                  // element of the 64 x 16 tile: k = e / 16, column j = e % 16
    const int kk = e >> 4, j = e & 15;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) sum += red[w][kk >> 2][(kk & 3) * 16 + j];
    if (k0 + kk < K && j < N) wp[static_cast<int64_t>(k0 + kk) * N + j] = sum;
  }
}

// out[k, j] (+)= sum over the row chunks of their partial products.  One warp per output element: lane l adds
// chunks l, l + 32, ... in that order, then the 32 lane sums are folded by a fixed shuffle tree -- the same order
// on every run.  (One thread per element walking all chunks took 56 us for a 16 x 41 product cut into 561 chunks.)
__global__ void __launch_bounds__(256)
gemm_tn_reduce_kernel(const float* __restrict__ ws, int chunks, int K, int N, float* __restrict__ out, int64_t ldo,
                      float beta, int transposed) {
  const int idx = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;      // warp-uniform
  const int lane = threadIdx.x & 31;
  if (idx >= K * N) return;
  float s = 0.f;
  for (int c = lane; c < chunks; c += 32) s += __ldg(ws + static_cast<int64_t>(c) * K * N + idx);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
  if (lane == 0) {
    // transposed: the partials are those of G^T * H (K and N as passed here); out is (H^T * G)[N x K]
    float* o = transposed ? out + static_cast<int64_t>(idx % N) * ldo + idx / N
                          : out + static_cast<int64_t>(idx / N) * ldo + idx % N;
    *o = (beta != 0.f) ? s + *o : s;
  }
}

struct TnShape {
  int chunks;
  int64_t rows_per_chunk;
  int ktiles, ntiles;
};

static TnShape tn_shape(int64_t n, int K, int N) {
  TnShape s;
  s.ktiles = (K + kTnKT - 1) / kTnKT;
  s.ntiles = (N + kTnNT - 1) / kTnNT;
  int64_t target = (4 * kNumSMs) / (static_cast<int64_t>(s.ktiles) * s.ntiles);
  if (target < 1) target = 1;
  const int64_t max_chunks = (n + 255) / 256;
  int64_t chunks = target < max_chunks ? target : max_chunks;
  if (chunks < 1) chunks = 1;
  int64_t rows = (n + chunks - 1) / chunks;
  rows = (rows + kTnRB - 1) / kTnRB * kTnRB;
  if (rows < kTnRB) rows = kTnRB;
  s.rows_per_chunk = rows;
  s.chunks = static_cast<int>((n + rows - 1) / rows);
  if (s.chunks < 1) s.chunks = 1;
  return s;
}

// ------------------------------------------------------------------------------------------------
__global__ void relu_fwd_kernel(const float* __restrict__ z, int64_t ldz, float* __restrict__ h, int64_t ldh, int64_t n,
                                int N) {
  const int64_t total = n * N;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / N;
    const int c = static_cast<int>(i - r * N);
    h[r * ldh + c] = fmaxf(z[r * ldz + c], 0.f);
  }
}

__global__ void relu_bwd_kernel(const float* __restrict__ h, int64_t ldh, const float* __restrict__ g, int64_t ldg,
                                float* __restrict__ dz, int64_t lddz, int64_t n, int N) {
  const int64_t total = n * N;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / N;
    const int c = static_cast<int>(i - r * N);
    dz[r * lddz + c] = h[r * ldh + c] > 0.f ? g[r * ldg + c] : 0.f;
  }
}

// one warp per row
__global__ void log_softmax_fwd_kernel(const float* __restrict__ z, int64_t ldz, float* __restrict__ out, int64_t ldo,
                                       int64_t n, int N) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  const float* zp = z + row * ldz;
  float mx = -INFINITY;
  for (int c = lane; c < N; c += 32) mx = fmaxf(mx, zp[c]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  float sum = 0.f;
  for (int c = lane; c < N; c += 32) sum += expf(zp[c] - mx);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  const float lse = mx + logf(sum);
  for (int c = lane; c < N; c += 32) out[row * ldo + c] = zp[c] - lse;
}

__global__ void log_softmax_bwd_kernel(const float* __restrict__ logp, int64_t ldl, const float* __restrict__ g,
                                       int64_t ldg, float* __restrict__ dz, int64_t lddz, int64_t n, int N) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  float sum = 0.f;
  for (int c = lane; c < N; c += 32) sum += g[row * ldg + c];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  for (int c = lane; c < N; c += 32) dz[row * lddz + c] = g[row * ldg + c] - expf(logp[row * ldl + c]) * sum;
}

// Pieces of a log-softmax whose rows are split over several processes: every process reduces its own
// columns, the per-row scalars are combined by a collective, then applied.   mode: 0 max, 1 sum,
// 2 sum of exp(z - ref[row]).  One warp per row.
__global__ void row_reduce_kernel(const float* __restrict__ z, int64_t ldz, int64_t n, int N, int mode,
                                  const float* __restrict__ ref, float* __restrict__ out) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  const float* zp = z + row * ldz;
  float acc = (mode == 0) ? -INFINITY : 0.f;
  const float r = (mode == 2) ? ref[row] : 0.f;
  for (int c = lane; c < N; c += 32) {
    const float v = zp[c];
    if (mode == 0) acc = fmaxf(acc, v);
    else if (mode == 1) acc += v;
    else acc += expf(v - r);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float o = __shfl_xor_sync(0xffffffffu, acc, off);
    acc = (mode == 0) ? fmaxf(acc, o) : acc + o;
  }
  if (lane == 0) out[row] = acc;
}

// mode 0: out = z - a[row] - log(b[row])        (log-softmax from the global row max a and sum b)
// mode 1: out = g - exp(z) * a[row]             (its backward from log-probabilities z and the global row sum a of g)
__global__ void row_apply_kernel(const float* __restrict__ z, int64_t ldz, const float* __restrict__ g, int64_t ldg,
                                 const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                                 int64_t ldo, int64_t n, int N, int mode) {
  const int64_t total = n * N;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / N;
    const int c = static_cast<int>(i - r * N);
    if (mode == 0) out[r * ldo + c] = z[r * ldz + c] - a[r] - logf(b[r]);
    else out[r * ldo + c] = g[r * ldg + c] - expf(z[r * ldz + c]) * a[r];
  }
}

// ------------------------------------------------------------------------------------------------
constexpr int kNllBlocks = 1024;

__global__ void __launch_bounds__(256) nll_partial_kernel(const float* __restrict__ logp, int64_t ldl,
                                                          const int64_t* __restrict__ y,
                                                          const uint8_t* __restrict__ mask, int64_t n, int N, int cls_lo,
                                                          int cls_hi, float gval, float* __restrict__ grad, int64_t ldg,
                                                          float* __restrict__ partial) {
  __shared__ float red[256];
  float s = 0.f;
  const int64_t total = n * N;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / N;
    const int c = static_cast<int>(i - r * N);
    const int64_t label = y[r];
    const bool hit = mask[r] && label >= cls_lo && label < cls_hi && (label - cls_lo) == c;
    if (hit) s += logp[r * ldl + c];
    if (grad) grad[r * ldg + c] = hit ? gval : 0.f;
  }
  red[threadIdx.x] = s;
  __syncthreads();
  for (int w = 128; w > 0; w >>= 1) {
    if (threadIdx.x < w) red[threadIdx.x] += red[threadIdx.x + w];
    __syncthreads();
  }
  if (threadIdx.x == 0) partial[blockIdx.x] = red[0];
}

__global__ void nll_final_kernel(const float* __restrict__ partial, int blocks, float count, float* __restrict__ loss) {
  __shared__ float red[256];
  float s = 0.f;
  for (int i = threadIdx.x; i < blocks; i += 256) s += partial[i];
  red[threadIdx.x] = s;
  __syncthreads();
  for (int w = 128; w > 0; w >>= 1) {
    if (threadIdx.x < w) red[threadIdx.x] += red[threadIdx.x + w];
    __syncthreads();
  }
  if (threadIdx.x == 0) *loss = -red[0] / count;
}

static int elementwise_blocks(int64_t total) {
  int64_t b = (total + 255) / 256;
  const int64_t cap = 32 * kNumSMs;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace cagnet

using namespace cagnet;

extern "C" int cagnet_gemm_nn_f32(const float* X, int64_t ldx, const float* W, int64_t ldw, int32_t transW, float* Z,
                                  int64_t ldz, int64_t n, int32_t K, int32_t N, int32_t epilogue, const float* aux,
                                  int64_t ldaux, void* stream) {
  if (n < 0 || K < 0 || N < 0) return fail(CAGNET_E_ARG, "cagnet_gemm_nn_f32: negative size");
  if (n == 0 || N == 0) return CAGNET_OK;
  if (!X || !W || !Z) return fail(CAGNET_E_ARG, "cagnet_gemm_nn_f32: null pointer");
  if (epilogue < 0 || epilogue > 4) return fail(CAGNET_E_ARG, "cagnet_gemm_nn_f32: unknown epilogue");
  if (epilogue == CAGNET_EPI_RELU_MASK && (!aux || ldaux < N))
    return fail(CAGNET_E_ARG, "cagnet_gemm_nn_f32: the ReLU-mask epilogue needs aux (n x N)");
  if (epilogue == CAGNET_EPI_LOG_SOFTMAX && N > 64)
    return fail(CAGNET_E_ARG, "cagnet_gemm_nn_f32: fused log-softmax supports N <= 64 (got %s%lld)", "", N);
  if (ldx < K || ldz < N || ldw < (transW ? K : N))
    return fail(CAGNET_E_ALIGN, "cagnet_gemm_nn_f32: leading dimension smaller than the row width");
  if ((n + kBM - 1) / kBM > INT_MAX) return fail(CAGNET_E_OVERFLOW, "cagnet_gemm_nn_f32: too many rows");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int x_vec4 = (ldx % 4 == 0 && aligned(X, 16)) ? 1 : 0;
  const unsigned gx = static_cast<unsigned>((n + kBM - 1) / kBM);
  const int per = N <= 64 ? (N + 7) / 8 : 8;   // columns per thread
#define CAGNET_GEMM_CASE(TN)                                                                                    \
  gemm_nn_kernel<TN><<<dim3(gx, (N + 8 * TN - 1) / (8 * TN)), 256, 0, s>>>(X, ldx, W, ldw, transW, Z, ldz, n, K, N, \
                                                                           epilogue, aux, ldaux, x_vec4)
  if (per <= 1) CAGNET_GEMM_CASE(1);
  else if (per <= 2) CAGNET_GEMM_CASE(2);
  else if (per <= 3) CAGNET_GEMM_CASE(3);
  else if (per <= 4) CAGNET_GEMM_CASE(4);
  else if (per <= 6) CAGNET_GEMM_CASE(6);
  else CAGNET_GEMM_CASE(8);
#undef CAGNET_GEMM_CASE
  return check_launch("cagnet_gemm_nn_f32");
}

extern "C" size_t cagnet_gemm_tn_workspace_bytes(int64_t n, int32_t K, int32_t N) {
  if (n < 0 || K <= 0 || N <= 0) return 0;
  const int chunks = max(tn_shape(n, K, N).chunks, tn_shape(n, N, K).chunks);     // either operand order
  return sizeof(float) * static_cast<size_t>(chunks) * K * N;
}

// The small-N kernel needs 80 KB of dynamic shared memory: opt in once per device.
static int tn_small_opt_in() {
  static bool opted_in[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !opted_in[dev]) {
    if (cudaFuncSetAttribute(gemm_tn_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTnSmallSmemBytes) !=
        cudaSuccess)
      return fail(CAGNET_E_LAUNCH, "cagnet_gemm_tn_f32: cannot reserve shared memory for the small-N kernel");
    opted_in[dev] = true;
  }
  return CAGNET_OK;
}

extern "C" int cagnet_gemm_tn_f32(const float* H, int64_t ldh, const float* G, int64_t ldg, float* out, int64_t ldo,
                                  int64_t n, int32_t K, int32_t N, float beta, void* ws, size_t ws_bytes, void* stream) {
  if (n < 0 || K < 0 || N < 0) return fail(CAGNET_E_ARG, "cagnet_gemm_tn_f32: negative size");
  if (K == 0 || N == 0) return CAGNET_OK;
  if (beta != 0.f && beta != 1.f) return fail(CAGNET_E_ARG, "cagnet_gemm_tn_f32: beta must be 0 or 1");
  if (!out || !ws || (n > 0 && (!H || !G))) return fail(CAGNET_E_ARG, "cagnet_gemm_tn_f32: null pointer");
  if (ldh < K || ldg < N || ldo < N) return fail(CAGNET_E_ALIGN, "cagnet_gemm_tn_f32: leading dimension too small");
  if (static_cast<int64_t>(K) * N > INT_MAX) return fail(CAGNET_E_OVERFLOW, "cagnet_gemm_tn_f32: K*N exceeds int32");
  if (ws_bytes < cagnet_gemm_tn_workspace_bytes(n, K, N))
    return fail(CAGNET_E_WORKSPACE, "cagnet_gemm_tn_f32: workspace of %s%lld bytes is too small (need %lld)", "",
                (long long)ws_bytes, (long long)cagnet_gemm_tn_workspace_bytes(n, K, N));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* partials = static_cast<float*>(ws);
  const bool rows_aligned = ldh % 4 == 0 && ldg % 4 == 0 && aligned(H, 16) && aligned(G, 16);
  if (N <= 16 && rows_aligned) {
    const TnShape sh = tn_shape(n, K, N);
    if (int rc = tn_small_opt_in()) return rc;
    gemm_tn_small_kernel<<<dim3(sh.chunks, sh.ktiles), 256, kTnSmallSmemBytes, s>>>(H, ldh, G, ldg, n, K, N,
                                                                                   sh.rows_per_chunk, partials);
    gemm_tn_reduce_kernel<<<(K * N + 7) / 8, 256, 0, s>>>(partials, sh.chunks, K, N, out, ldo, beta, 0);
  } else if (K <= 16 && rows_aligned) {
    // a narrow H against a wider G (the 16 x 41 weight gradient): the same kernel computes G^T * H, the reduce
    // writes it transposed
    const TnShape sh = tn_shape(n, N, K);
    if (int rc = tn_small_opt_in()) return rc;
    gemm_tn_small_kernel<<<dim3(sh.chunks, sh.ktiles), 256, kTnSmallSmemBytes, s>>>(G, ldg, H, ldh, n, N, K,
                                                                                   sh.rows_per_chunk, partials);
    gemm_tn_reduce_kernel<<<(K * N + 7) / 8, 256, 0, s>>>(partials, sh.chunks, N, K, out, ldo, beta, 1);
  } else {
    const TnShape sh = tn_shape(n, K, N);
    gemm_tn_partial_kernel<<<dim3(sh.chunks, sh.ktiles, sh.ntiles), 256, 0, s>>>(H, ldh, G, ldg, n, K, N,
                                                                                sh.rows_per_chunk, partials);
    gemm_tn_reduce_kernel<<<(K * N + 7) / 8, 256, 0, s>>>(partials, sh.chunks, K, N, out, ldo, beta, 0);
  }
  return check_launch("cagnet_gemm_tn_f32");
}

extern "C" int cagnet_relu_fwd_f32(const float* z, int64_t ldz, float* h, int64_t ldh, int64_t n, int32_t N,
                                   void* stream) {
  if (n < 0 || N < 0) return fail(CAGNET_E_ARG, "cagnet_relu_fwd_f32: negative size");
  if (n == 0 || N == 0) return CAGNET_OK;
  if (!z || !h || ldz < N || ldh < N) return fail(CAGNET_E_ARG, "cagnet_relu_fwd_f32: bad argument");
  relu_fwd_kernel<<<elementwise_blocks(n * N), 256, 0, static_cast<cudaStream_t>(stream)>>>(z, ldz, h, ldh, n, N);
  return check_launch("cagnet_relu_fwd_f32");
}

extern "C" int cagnet_relu_bwd_f32(const float* h, int64_t ldh, const float* g, int64_t ldg, float* dz, int64_t lddz,
                                   int64_t n, int32_t N, void* stream) {
  if (n < 0 || N < 0) return fail(CAGNET_E_ARG, "cagnet_relu_bwd_f32: negative size");
  if (n == 0 || N == 0) return CAGNET_OK;
  if (!h || !g || !dz || ldh < N || ldg < N || lddz < N) return fail(CAGNET_E_ARG, "cagnet_relu_bwd_f32: bad argument");
  relu_bwd_kernel<<<elementwise_blocks(n * N), 256, 0, static_cast<cudaStream_t>(stream)>>>(h, ldh, g, ldg, dz, lddz, n, N);
  return check_launch("cagnet_relu_bwd_f32");
}

extern "C" int cagnet_log_softmax_fwd_f32(const float* z, int64_t ldz, float* logp, int64_t ldl, int64_t n, int32_t N,
                                          void* stream) {
  if (n < 0 || N < 0) return fail(CAGNET_E_ARG, "cagnet_log_softmax_fwd_f32: negative size");
  if (n == 0 || N == 0) return CAGNET_OK;
  if (!z || !logp || ldz < N || ldl < N) return fail(CAGNET_E_ARG, "cagnet_log_softmax_fwd_f32: bad argument");
  if ((n + 7) / 8 > INT_MAX) return fail(CAGNET_E_OVERFLOW, "cagnet_log_softmax_fwd_f32: too many rows");
  log_softmax_fwd_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(z, ldz, logp,
                                                                                                          ldl, n, N);
  return check_launch("cagnet_log_softmax_fwd_f32");
}

extern "C" int cagnet_log_softmax_bwd_f32(const float* logp, int64_t ldl, const float* g, int64_t ldg, float* dz,
                                          int64_t lddz, int64_t n, int32_t N, void* stream) {
  if (n < 0 || N < 0) return fail(CAGNET_E_ARG, "cagnet_log_softmax_bwd_f32: negative size");
  if (n == 0 || N == 0) return CAGNET_OK;
  if (!logp || !g || !dz || ldl < N || ldg < N || lddz < N)
    return fail(CAGNET_E_ARG, "cagnet_log_softmax_bwd_f32: bad argument");
  if ((n + 7) / 8 > INT_MAX) return fail(CAGNET_E_OVERFLOW, "cagnet_log_softmax_bwd_f32: too many rows");
  log_softmax_bwd_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      logp, ldl, g, ldg, dz, lddz, n, N);
  return check_launch("cagnet_log_softmax_bwd_f32");
}

extern "C" int cagnet_row_reduce_f32(const float* z, int64_t ldz, int64_t n, int32_t N, int32_t mode, const float* ref,
                                     float* out, void* stream) {
  if (n < 0 || N < 0) return fail(CAGNET_E_ARG, "cagnet_row_reduce_f32: negative size");
  if (n == 0) return CAGNET_OK;
  if (mode < 0 || mode > 2 || !out || (N > 0 && !z) || (mode == 2 && !ref) || ldz < N)
    return fail(CAGNET_E_ARG, "cagnet_row_reduce_f32: bad argument");
  if ((n + 7) / 8 > INT_MAX) return fail(CAGNET_E_OVERFLOW, "cagnet_row_reduce_f32: too many rows");
  row_reduce_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(z, ldz, n, N, mode,
                                                                                                     ref, out);
  return check_launch("cagnet_row_reduce_f32");
}

extern "C" int cagnet_log_softmax_apply_f32(const float* z, int64_t ldz, const float* row_max, const float* row_sum,
                                            float* logp, int64_t ldl, int64_t n, int32_t N, void* stream) {
  if (n < 0 || N < 0) return fail(CAGNET_E_ARG, "cagnet_log_softmax_apply_f32: negative size");
  if (n == 0 || N == 0) return CAGNET_OK;
  if (!z || !row_max || !row_sum || !logp || ldz < N || ldl < N)
    return fail(CAGNET_E_ARG, "cagnet_log_softmax_apply_f32: bad argument");
  row_apply_kernel<<<elementwise_blocks(n * N), 256, 0, static_cast<cudaStream_t>(stream)>>>(z, ldz, nullptr, 0, row_max,
                                                                                           row_sum, logp, ldl, n, N, 0);
  return check_launch("cagnet_log_softmax_apply_f32");
}

extern "C" int cagnet_log_softmax_bwd_apply_f32(const float* logp, int64_t ldl, const float* g, int64_t ldg,
                                                const float* row_sum_g, float* dz, int64_t lddz, int64_t n, int32_t N,
                                                void* stream) {
  if (n < 0 || N < 0) return fail(CAGNET_E_ARG, "cagnet_log_softmax_bwd_apply_f32: negative size");
  if (n == 0 || N == 0) return CAGNET_OK;
  if (!logp || !g || !row_sum_g || !dz || ldl < N || ldg < N || lddz < N)
    return fail(CAGNET_E_ARG, "cagnet_log_softmax_bwd_apply_f32: bad argument");
  row_apply_kernel<<<elementwise_blocks(n * N), 256, 0, static_cast<cudaStream_t>(stream)>>>(logp, ldl, g, ldg, row_sum_g,
                                                                                           nullptr, dz, lddz, n, N, 1);
  return check_launch("cagnet_log_softmax_bwd_apply_f32");
}

extern "C" size_t cagnet_nll_workspace_bytes(int64_t n) {
  (void)n;
  return sizeof(float) * kNllBlocks;
}

extern "C" int cagnet_nll_masked_f32(const float* logp, int64_t ldl, const int64_t* y, const uint8_t* mask, int64_t n,
                                     int32_t N, int32_t cls_lo, int32_t cls_hi, float count, float scale,
                                     float* loss_dev, float* grad, int64_t ldg, void* ws, size_t ws_bytes,
                                     void* stream) {
  if (n < 0 || N <= 0) return fail(CAGNET_E_ARG, "cagnet_nll_masked_f32: bad size");
  if (!loss_dev || !ws || (n > 0 && (!logp || !y || !mask))) return fail(CAGNET_E_ARG, "cagnet_nll_masked_f32: null pointer");
  if (ldl < N || (grad && ldg < N)) return fail(CAGNET_E_ALIGN, "cagnet_nll_masked_f32: leading dimension too small");
  if (ws_bytes < cagnet_nll_workspace_bytes(n)) return fail(CAGNET_E_WORKSPACE, "cagnet_nll_masked_f32: workspace too small");
  if (!(count > 0.f)) return fail(CAGNET_E_ARG, "cagnet_nll_masked_f32: count must be positive");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int blocks = elementwise_blocks(n * N);
  if (blocks > kNllBlocks) blocks = kNllBlocks;
  nll_partial_kernel<<<blocks, 256, 0, s>>>(logp, ldl, y, mask, n, N, cls_lo, cls_hi, -scale / count, grad, ldg,
                                            static_cast<float*>(ws));
  nll_final_kernel<<<1, 256, 0, s>>>(static_cast<const float*>(ws), blocks, count, loss_dev);
  return check_launch("cagnet_nll_masked_f32");
}
