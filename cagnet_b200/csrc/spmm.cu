// Row-split CSR SpMM for sm_100a:  C = beta*C + A*B,  fp32 values, int32 indices, row-major B and C.
//
// Work decomposition
//   * one warp per CSR row for ordinary rows; the warp reads the row's (col, val) pairs 32 at a
//     time with one coalesced load per array and shares them through a 256-byte shared-memory stage;
//   * LPN lanes cover one gathered row of B with VEC-wide vectors (VEC = 4 -> 128-bit loads), so a
//     warp works on 32/LPN nonzeros at once: narrow B (f = 16) keeps all 32 lanes busy;
//   * NV vectors per lane make a feature tile of LPN*VEC*NV columns; wider B is covered by
//     gridDim.y tiles, dispatched tile-major so that one column slab of B stays hot in L2;
//   * rows longer than the plan's threshold (power-law hubs) are taken out of the warp-per-row
//     pass and processed by a whole 512-thread block each, 16 warps on disjoint nonzero ranges,
//     combined through shared memory in warp order;
//   * blocks with short rows (few nonzeros per row on average) and a narrow B run the lane-group kernel
//     instead of the warp-per-row one: a warp owns a pool of up to 32 consecutive rows, each of its 32/LPN
//     lane groups walks one short row at a time and takes the next unclaimed row of the pool when it is
//     done, so no lane waits for a whole warp's fixed cost per 5-nonzero row; the pool's longer rows are
//     then multiplied by the whole warp as in the warp-per-row kernel.
// Every output element is produced by a fixed sequence of operations: results are bit-reproducible
// run to run, no floating-point atomics anywhere.
#include <limits.h>

#include "common.cuh"

namespace cagnet {

struct Tuning {
  int spmm_tile = 0;     // vectors per feature tile: 0 = automatic, else 4, 8, 16, 32, 64, 96, 128 or 160
  int spmm_rpb = 4;      // rows (warps) per thread block of the warp-per-row kernel: 1, 2, 4 or 8
  int spmm_long = 2048;         // rows with more nonzeros are listed in the plan (block-per-row kernel)
  int spmm_long_narrow = 2048;  // products narrower than 32 vectors may keep more rows in the warp-per-row pass
  int spmm_group_max = 64;      // lane-group kernel: rows up to this length are walked by one lane group
  int spmm_group_avg = 96;      // blocks with at most this many nonzeros per row on average use it (0 = never)
  int spmm_group_pool = 0;      // rows per warp pool there: 0 = automatic, else 4, 8, 16 or 32
  int spmm_overlap = 1;         // the row kernel may start under the hub-row kernel's tail (programmatic launch)
  int spmm_deep = 1;            // narrow B: gathers issued in batches of 4-8 per lane before their FMAs
};
static Tuning g_tuning;

constexpr int kPlanMagic = 0x0CA67E70;
constexpr int kPlanHeaderInts = 8;   // [0] magic [1] count [2] threshold [3] capacity
constexpr int kMinLongThreshold = 256;
constexpr int kLongWarps = 16;
// (col, val) pairs a warp parks in shared memory at a time: 32, or 64 where gathers are batched with 4 lanes per
// nonzero (a batch of 8 per lane group needs 64 pairs).  Kept as small as the variant allows: shared memory is carved
// out of the L1 cache, and the wide, bandwidth-bound products lost 5 % when every variant reserved 64.
template <int LPN, bool DEEP>
struct StagePairs {
  static constexpr int value = (DEEP && LPN <= 4) ? 64 : 32;
};

// ------------------------------------------------------------------------------------------------
template <int VEC>
__device__ __forceinline__ void load_vec(const float* __restrict__ p, float (&x)[VEC]) {
  if constexpr (VEC == 4) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(p));
    x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w;
  } else if constexpr (VEC == 2) {
    const float2 t = __ldg(reinterpret_cast<const float2*>(p));
    x[0] = t.x; x[1] = t.y;
  } else {
    x[0] = __ldg(p);
  }
}

template <int VEC>
__device__ __forceinline__ void store_vec(float* p, const float (&x)[VEC]) {
  if constexpr (VEC == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
  } else if constexpr (VEC == 2) {
    *reinterpret_cast<float2*>(p) = make_float2(x[0], x[1]);
  } else {
    *p = x[0];
  }
}

// Stores the leading `live` (<= VEC) elements of x: the vector that straddles the matrix's last column is written
// element by element, so that columns [f, ld) of C -- which may belong to the caller -- are never touched.
template <int VEC>
__device__ __forceinline__ void store_vec_upto(float* p, const float (&x)[VEC], int live) {
  if (live >= VEC) {
    store_vec<VEC>(p, x);
  } else {
#pragma unroll
    for (int j = 0; j < VEC; ++j)
      if (j < live) p[j] = x[j];
  }
}

// C[row, tile columns of this lane] = acc (+ the old value when beta != 0), columns >= f left alone.
template <int VEC, int LPN, int NV>
__device__ __forceinline__ void store_row(float* __restrict__ cp, int column0, int f, int nvalid, float beta,
                                          float (&acc)[NV][VEC]) {
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    if (k < nvalid) {
      const int live = f - (column0 + k * (LPN * VEC));
      if (live <= 0) continue;
      if (beta != 0.f) {
        float old[VEC];
        load_vec<VEC>(cp + k * (LPN * VEC), old);      // inside the padded row: reading is harmless
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[k][j] += old[j];
      }
      store_vec_upto<VEC>(cp + k * (LPN * VEC), acc[k], live);
    }
  }
}

// The hub-row kernel and the row kernel of one multiply write disjoint rows of C, so they may overlap: the hub
// kernel's longest row (100K+ nonzeros in an R-MAT graph, one thread block) would otherwise be a tail during which
// the rest of the GPU idles.  The row kernel is launched with programmatic stream serialisation: it may start as
// soon as every block of the hub kernel has begun (`pdl_release_dependents`), and it does not complete before the
// hub kernel has (`pdl_waiter_block`), so that whatever follows in the stream
// still sees both kernels finished.  The waiting is done by ONE EXTRA block appended to the row kernel's grid, which
// does nothing else: a grid is complete when all its blocks are, so one waiting block is enough to order the
// completions, and the working blocks leave at once instead of holding their SM slots until the hub kernel's last
// row is done.  (Waiting at the end of a working block instead cost the row kernel 6 registers, 38 for 32, and with
// them a quarter of its resident warps.)
__device__ __forceinline__ void pdl_release_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
// True for the appended block: its first thread waits for the hub kernel, all its threads then leave.
__device__ __forceinline__ bool pdl_waiter_block(int waiter) {
  if (!waiter || blockIdx.x != gridDim.x - 1) return false;
  if (blockIdx.y == 0 && threadIdx.x == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
  return true;
}

// Accumulates sum_e val[e] * B[col[e], tile columns of this lane] over e in [start, end) into acc.
// bt already points at column (tile0 + l*VEC) of row 0 of B; vector k of the lane sits k*LPN*VEC columns
// further on and is live iff k < nvalid.
//
// The warp reads 32 (col, val) pairs with two coalesced loads and parks them in its 256-byte slice of shared
// memory (`stage`); every lane then needs every pair, and gets two of them per 128-bit broadcast read.  Per
// nonzero and warp that leaves half a shared-memory read, one widening multiply-add for the row address, one
// 128-bit gather and the FMAs -- the first version handed the pairs round with two warp shuffles per nonzero
// and a 64-bit multiply, 22 instructions per nonzero, and ran at half of the issue rate without saturating
// either L2 or HBM.
//
// Narrow B (LPN < 32, several lane groups per warp) is bound by memory latency, not bandwidth: a gathered row is
// 64-256 bytes and nothing else keeps the warp busy while it travels.  There the pairs of a chunk are consumed in
// batches: the batch's pairs are read from shared memory, then ALL its gathers are issued into registers, and only
// then do the FMAs run (in nonzero order, so the sums are the same numbers as one gather at a time would give).
// A lane then has 4-8 independent 128-bit gathers in flight instead of whatever the compiler chose to overlap; with
// 4 lanes per nonzero a chunk is 64 pairs, so that a batch of 8 exists.
template <int VEC, int LPN, int NV>
__device__ __forceinline__ void accumulate_range_batched(const int* __restrict__ col, const float* __restrict__ val,
                                                         int start, int end, const float* __restrict__ bt, int ldb,
                                                         int nvalid, int lane, int2* stage, float (&acc)[NV][VEC]) {
  static_assert(LPN < 32, "batched gathers are for narrow B");
  constexpr int G = 32 / LPN;
  constexpr int CH = (LPN <= 4) ? 64 : 32;         // pairs staged per chunk
  constexpr int PER = CH / G;                      // pairs one lane group consumes per chunk
  constexpr int BATCH = (NV >= 2) ? 4 : 8;         // gathers in flight per lane
  static_assert(PER % BATCH == 0 && CH == StagePairs<LPN, true>::value, "chunk / batch mismatch");
  const int sub = lane / LPN;
  auto load_pair = [&](int e) {
    int2 p = make_int2(0, 0);
    if (e < end) {
      p.x = __ldg(col + e);
      p.y = __float_as_int(__ldg(val + e));
    }
    return p;
  };
  int2 next0 = load_pair(start + lane), next1 = make_int2(0, 0);
  if constexpr (CH == 64) next1 = load_pair(start + 32 + lane);
  for (int base = start; base < end; base += CH) {
    __syncwarp();            // every lane is done with the previous chunk
    stage[lane] = next0;
    if constexpr (CH == 64) stage[32 + lane] = next1;
    __syncwarp();
    next0 = load_pair(base + CH + lane);           // the following chunk's pairs travel while this one is gathered
    if constexpr (CH == 64) next1 = load_pair(base + CH + 32 + lane);
    const int cnt = min(CH, end - base);
#pragma unroll
    for (int b = 0; b < PER; b += BATCH) {
      if (b * G >= cnt) break;                     // warp-uniform
      int c[BATCH];
      float v[BATCH];
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int idx = (b + i) * G + sub;
        const int2 q = stage[min(idx, CH - 1)];
        c[i] = idx < cnt ? q.x : -1;
        v[i] = idx < cnt ? __int_as_float(q.y) : 0.f;
      }
      float x[BATCH][NV][VEC];
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const float* bp = bt + static_cast<int64_t>(c[i] < 0 ? 0 : c[i]) * ldb;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
          if (c[i] >= 0 && k < nvalid) {
            load_vec<VEC>(bp + k * (LPN * VEC), x[i][k]);
          } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) x[i][k][j] = 0.f;
          }
        }
      }
#pragma unroll
      for (int i = 0; i < BATCH; ++i)
#pragma unroll
        for (int k = 0; k < NV; ++k)
#pragma unroll
          for (int j = 0; j < VEC; ++j) acc[k][j] = fmaf(v[i], x[i][k][j], acc[k][j]);
    }
  }
  // fold the 32/LPN nonzero slots of the warp together; afterwards every lane holds the row sums
#pragma unroll
  for (int off = LPN; off < 32; off <<= 1) {
#pragma unroll
    for (int k = 0; k < NV; ++k)
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[k][j] += __shfl_xor_sync(0xffffffffu, acc[k][j], off);
  }
}

template <int VEC, int LPN, int NV, bool DEEP = false>
__device__ __forceinline__ void accumulate_range(const int* __restrict__ col, const float* __restrict__ val,
                                                 int start, int end, const float* __restrict__ bt, int ldb,
                                                 int nvalid, int lane, int2* stage, float (&acc)[NV][VEC]) {
  if constexpr (DEEP && LPN < 32) {
    accumulate_range_batched<VEC, LPN, NV>(col, val, start, end, bt, ldb, nvalid, lane, stage, acc);
    return;
  }
  constexpr int G = 32 / LPN;                      // nonzeros in flight per warp step
#ifndef CAGNET_SPMM_UNROLL
#define CAGNET_SPMM_UNROLL 8
#endif
  constexpr int UNROLL = (NV >= 4) ? 1 : (NV >= 2 ? 2 : CAGNET_SPMM_UNROLL);
  const int sub = lane / LPN;

  auto gather = [&](int c, float v) {
    const float* bp = bt + static_cast<int64_t>(c) * ldb;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      if (k < nvalid) {
        float x[VEC];
        load_vec<VEC>(bp + k * (LPN * VEC), x);
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[k][j] = fmaf(v, x[j], acc[k][j]);
      }
    }
  };

  auto load_pair = [&](int e) {
    int2 p = make_int2(0, 0);
    if (e < end) {
      p.x = __ldg(col + e);
      p.y = __float_as_int(__ldg(val + e));
    }
    return p;
  };
  int2 next = load_pair(start + lane);
  for (int base = start; base < end; base += 32) {
    __syncwarp();            // every lane is done with the previous chunk
    stage[lane] = next;
    __syncwarp();
    next = load_pair(base + 32 + lane);   // the following chunk's pairs travel while this one is being gathered
    const int cnt = min(32, end - base);
    if (cnt == 32) {
      if constexpr (G == 1) {
#pragma unroll UNROLL
        for (int s = 0; s < 32; s += 2) {
          const int4 q = *reinterpret_cast<const int4*>(stage + s);
          gather(q.x, __int_as_float(q.y));
          gather(q.z, __int_as_float(q.w));
        }
      } else {
#pragma unroll 4
        for (int s = 0; s < 32; s += G) {
          const int2 q = stage[s + sub];
          gather(q.x, __int_as_float(q.y));
        }
      }
    } else {
      for (int s = 0; s < cnt; s += G) {
        if (s + sub < cnt) {
          const int2 q = stage[s + sub];
          gather(q.x, __int_as_float(q.y));
        }
      }
    }
  }
  // fold the 32/LPN nonzero slots of the warp together; afterwards every lane holds the row sums
#pragma unroll
  for (int off = LPN; off < 32; off <<= 1) {
#pragma unroll
    for (int k = 0; k < NV; ++k)
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[k][j] += __shfl_xor_sync(0xffffffffu, acc[k][j], off);
  }
}

// live vectors of lane l in feature tile `tile`: columns tile0 + (k*LPN + l)*VEC < f_eff
template <int VEC, int LPN, int NV>
__device__ __forceinline__ int live_vectors(int tile0, int l, int f_eff) {
  const int first = tile0 + l * VEC;
  if (first >= f_eff) return 0;
  return min(NV, (f_eff - first + LPN * VEC - 1) / (LPN * VEC));
}

constexpr int kMaxRowsPerBlock = 8;

// (Holding this kernel to 32 registers with a second launch-bounds argument, for 64 instead of 48 resident warps per
// SM, measured 5-7 % SLOWER on the wide, memory-bound products: the compiler pays for the registers with serialised
// loads.)
template <int VEC, int LPN, int NV, bool DEEP>
__global__ void __launch_bounds__(kMaxRowsPerBlock * 32) spmm_warp_rows_kernel(
    const int* __restrict__ rowptr, const int* __restrict__ col, const float* __restrict__ val, int n,
    const float* __restrict__ B, int ldb, float* __restrict__ C, int ldc, int f_eff, int f, float beta,
    const int* __restrict__ plan, int min_threshold, int waiter) {
  __shared__ __align__(16) int2 stage[kMaxRowsPerBlock][StagePairs<LPN, DEEP>::value];
  if (pdl_waiter_block(waiter)) return;
  const int warp = threadIdx.x >> 5;
  const int row = blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= n) return;                      // whole warps leave together; nothing below is block-wide
  const int lane = threadIdx.x & 31;
  const int l = lane % LPN;
  const int tile0 = blockIdx.y * (LPN * VEC * NV);
  const int start = __ldg(rowptr + row);
  const int end = __ldg(rowptr + row + 1);
  const int long_threshold = plan ? max(__ldg(plan + 2), min_threshold) : INT_MAX;
  if (end - start > long_threshold) return;  // a hub row: the block-per-row kernel owns it
  const int nvalid = live_vectors<VEC, LPN, NV>(tile0, l, f_eff);

  float acc[NV][VEC];
#pragma unroll
  for (int k = 0; k < NV; ++k)
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[k][j] = 0.f;

  accumulate_range<VEC, LPN, NV, DEEP>(col, val, start, end, B + tile0 + l * VEC, ldb, nvalid, lane, stage[warp], acc);

  if (lane < LPN)
    store_row<VEC, LPN, NV>(C + static_cast<int64_t>(row) * ldc + tile0 + l * VEC, tile0 + l * VEC, f, nvalid, beta, acc);
}

// ------------------------------------------------------------------------------------------------
// Lane-group kernel for blocks of short rows (LPN < 32).
//
// A warp owns a pool of `pool` (<= 32) consecutive rows; lane i keeps row i's [start, end).  Rows are sorted
// into three classes by length alone, so the arithmetic of a row never depends on scheduling:
//   short   (<= group_max nonzeros): walked by ONE lane group (LPN lanes, each VEC*NV output columns), nonzero
//           after nonzero in order, UNROLL gathers in flight per group; a group that finishes takes the next
//           unclaimed short row of the pool (ballot + bit tricks, no memory traffic), so the 32/LPN groups stay
//           busy although their rows differ in length;
//   medium  (<= the plan's hub threshold): multiplied by the whole warp exactly as in the warp-per-row kernel
//           (pairs staged through shared memory, lane groups on interleaved nonzeros, shuffle fold);
//   hub     rows are skipped: the block-per-row kernel owns them.
// Per short row this costs a few instructions of bookkeeping instead of a warp's offsets load, stage, two
// warp barriers and a shuffle tree.
template <int VEC, int LPN, int NV, bool DEEP>
__global__ void __launch_bounds__(kMaxRowsPerBlock * 32) spmm_group_rows_kernel(
    const int* __restrict__ rowptr, const int* __restrict__ col, const float* __restrict__ val, int n,
    const float* __restrict__ B, int ldb, float* __restrict__ C, int ldc, int f_eff, int f, float beta,
    const int* __restrict__ plan, int min_threshold, int group_max, int pool, int waiter) {
  static_assert(LPN < 32, "the lane-group kernel needs at least two groups per warp");
  if (pdl_waiter_block(waiter)) return;
  constexpr int G = 32 / LPN;
#ifndef CAGNET_GROUP_UNROLL
#define CAGNET_GROUP_UNROLL 8
#endif
  constexpr int UNROLL = (NV >= 2) ? CAGNET_GROUP_UNROLL / 2 : CAGNET_GROUP_UNROLL;
  __shared__ __align__(16) int2 stage[kMaxRowsPerBlock][StagePairs<LPN, DEEP>::value];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int row0 = (blockIdx.x * (blockDim.x >> 5) + warp) * pool;
  if (row0 >= n) return;                      // whole warps leave together; nothing below is block-wide
  const int l = lane % LPN;
  const int sub = lane / LPN;
  const int tile0 = blockIdx.y * (LPN * VEC * NV);
  const int column0 = tile0 + l * VEC;
  const int nvalid = live_vectors<VEC, LPN, NV>(tile0, l, f_eff);
  const float* bt = B + column0;
  const int long_threshold = plan ? max(__ldg(plan + 2), min_threshold) : INT_MAX;

  // lane i: offsets of row row0 + i
  const bool have = lane < pool && row0 + lane < n;
  const int my_start = have ? __ldg(rowptr + row0 + lane) : 0;
  const int my_end = have ? __ldg(rowptr + row0 + lane + 1) : 0;
  const int my_len = my_end - my_start;
  const int short_max = min(group_max, long_threshold);      // longer rows belong to the warp or to the hub kernel
  unsigned pending = __ballot_sync(0xffffffffu, have && my_len <= short_max);
  unsigned medium = __ballot_sync(0xffffffffu, have && my_len > short_max && my_len <= long_threshold);

  float acc[NV][VEC];
  int cur = -1, e = 0, e_end = 0;             // the group's row (pool index) and its nonzero cursor
  for (;;) {
    const bool need = e >= e_end;             // uniform inside a lane group
    if (need && cur >= 0) {
      // every lane of the group holds its own columns of the row
      store_row<VEC, LPN, NV>(C + static_cast<int64_t>(row0 + cur) * ldc + column0, column0, f, nvalid, beta, acc);
      cur = -1;
    }
    // groups without a row claim the pool's next short rows, lowest group first
    const unsigned need_lanes = __ballot_sync(0xffffffffu, need);
    if (need_lanes) {
      unsigned groups = 0;                    // bit g: lane group g wants a row
#pragma unroll
      for (int g = 0; g < G; ++g) groups |= ((need_lanes >> (g * LPN)) & 1u) << g;
      const int rank = __popc(groups & ((1u << sub) - 1u));
      unsigned mine = pending;
      for (int i = 0; i < rank; ++i) mine &= mine - 1;            // drop the rows taken by lower groups
      const int pick = (need && mine) ? __ffs(mine) - 1 : -1;
      for (int i = __popc(groups); i > 0 && pending; --i) pending &= pending - 1;
      const int src = pick < 0 ? 0 : pick;
      const int s_new = __shfl_sync(0xffffffffu, my_start, src);
      const int e_new = __shfl_sync(0xffffffffu, my_end, src);
      if (need) {
        cur = pick;
        e = pick < 0 ? 0 : s_new;
        e_end = pick < 0 ? 0 : e_new;
#pragma unroll
        for (int k = 0; k < NV; ++k)
#pragma unroll
          for (int j = 0; j < VEC; ++j) acc[k][j] = 0.f;
      }
      if (__ballot_sync(0xffffffffu, cur >= 0) == 0) break;      // pool exhausted and every group is done
    }
    // up to UNROLL nonzeros of the group's row: offsets first, then the gathers, then the FMAs in order
    int c[UNROLL];
    float v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const bool ok = e + u < e_end;
      c[u] = ok ? __ldg(col + e + u) : -1;
      v[u] = ok ? __ldg(val + e + u) : 0.f;
    }
    float x[UNROLL][NV][VEC];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const float* bp = bt + static_cast<int64_t>(c[u] < 0 ? 0 : c[u]) * ldb;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        if (c[u] >= 0 && k < nvalid) {
          load_vec<VEC>(bp + k * (LPN * VEC), x[u][k]);
        } else {
#pragma unroll
          for (int j = 0; j < VEC; ++j) x[u][k][j] = 0.f;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int k = 0; k < NV; ++k)
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[k][j] = fmaf(v[u], x[u][k][j], acc[k][j]);
    e = min(e + UNROLL, e_end);
  }

  // the pool's medium rows, one after the other, by the whole warp
  while (medium) {
    const int i = __ffs(medium) - 1;
    medium &= medium - 1;
    const int start = __shfl_sync(0xffffffffu, my_start, i);
    const int end = __shfl_sync(0xffffffffu, my_end, i);
#pragma unroll
    for (int k = 0; k < NV; ++k)
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[k][j] = 0.f;
    accumulate_range<VEC, LPN, NV, DEEP>(col, val, start, end, bt, ldb, nvalid, lane, stage[warp], acc);
    if (lane < LPN)
      store_row<VEC, LPN, NV>(C + static_cast<int64_t>(row0 + i) * ldc + column0, column0, f, nvalid, beta, acc);
  }
}

template <int VEC, int LPN, int NV, bool DEEP>
__global__ void __launch_bounds__(kLongWarps * 32) spmm_block_rows_kernel(
    const int* __restrict__ rowptr, const int* __restrict__ col, const float* __restrict__ val,
    const float* __restrict__ B, int ldb, float* __restrict__ C, int ldc, int f_eff, int f, float beta,
    const int* __restrict__ plan, int min_threshold) {
  constexpr int TILE = LPN * VEC * NV;
  __shared__ float part[kLongWarps][TILE];
  __shared__ __align__(16) int2 stage[kLongWarps][StagePairs<LPN, DEEP>::value];
  pdl_release_dependents();
  const int long_threshold = max(__ldg(plan + 2), min_threshold);
  const int count = min(__ldg(plan + 1), __ldg(plan + 3));
  const int* list = plan + kPlanHeaderInts;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int l = lane % LPN;
  const int tile0 = blockIdx.y * TILE;
  const int nvalid = live_vectors<VEC, LPN, NV>(tile0, l, f_eff);

  for (int item = blockIdx.x; item < count; item += gridDim.x) {
    const int row = __ldg(list + item);
    const int start = __ldg(rowptr + row);
    const int end = __ldg(rowptr + row + 1);
    if (end - start <= long_threshold) continue;   // listed, but short enough for the warp-per-row pass at this width
    constexpr int PAIRS = StagePairs<LPN, DEEP>::value;
    const int per = (((end - start) + kLongWarps - 1) / kLongWarps + PAIRS - 1) & ~(PAIRS - 1);
    const int ws = min(end, start + warp * per);
    const int we = min(end, ws + per);

    float acc[NV][VEC];
#pragma unroll
    for (int k = 0; k < NV; ++k)
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[k][j] = 0.f;
    accumulate_range<VEC, LPN, NV, DEEP>(col, val, ws, we, B + tile0 + l * VEC, ldb, nvalid, lane, stage[warp], acc);

    if (lane < LPN) {
#pragma unroll
      for (int k = 0; k < NV; ++k)
#pragma unroll
        for (int j = 0; j < VEC; ++j) part[warp][(k * LPN + l) * VEC + j] = acc[k][j];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < TILE; idx += blockDim.x) {
      const int column = tile0 + idx;
      if (column < f) {
        float s = part[0][idx];
#pragma unroll
        for (int w = 1; w < kLongWarps; ++w) s += part[w][idx];
        float* cp = C + static_cast<int64_t>(row) * ldc + column;
        if (beta != 0.f) s += *cp;
        *cp = s;
      }
    }
    __syncthreads();
  }
}

// Appends the rows with lo < nonzeros <= hi to the plan's list.
__global__ void spmm_plan_kernel(const int* __restrict__ rowptr, int n, int lo, int hi, int capacity, int* plan) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n) return;
  const int len = rowptr[row + 1] - rowptr[row];
  if (len > lo && len <= hi) {
    const int slot = atomicAdd(plan + 1, 1);
    if (slot < capacity) plan[kPlanHeaderInts + slot] = row;
  }
}

// The list is filled longest rows first (four length classes, one pass each): the block-per-row kernel walks it
// in order, and a 100K-nonzero row that starts last would be the tail of the whole launch.
static void launch_plan_passes(const int* rowptr, int n, int threshold, int capacity, int* plan, cudaStream_t s) {
  const int64_t t = threshold;
  const int64_t cuts[5] = {INT_MAX, 32 * t, 8 * t, 2 * t, t};
  for (int pass = 0; pass < 4; ++pass) {
    const int hi = static_cast<int>(cuts[pass] > INT_MAX ? INT_MAX : cuts[pass]);
    const int lo = static_cast<int>(cuts[pass + 1] > INT_MAX ? INT_MAX : cuts[pass + 1]);
    if (lo >= hi) continue;
    spmm_plan_kernel<<<(n + 255) / 256, 256, 0, s>>>(rowptr, n, lo, hi, capacity, plan);
  }
}

__global__ void spmm_plan_header_kernel(int threshold, int capacity, int* plan) {
  plan[0] = kPlanMagic;
  plan[1] = 0;
  plan[2] = threshold;
  plan[3] = capacity;
}

static int plan_capacity(int64_t nnz, int threshold) { return static_cast<int>(nnz / threshold) + 1; }

// Rows per pool of the lane-group kernel: 32 when that still leaves every SM a few dozen warps, fewer for small blocks.
static int group_pool_rows(int n) {
  if (g_tuning.spmm_group_pool > 0) return g_tuning.spmm_group_pool;
  const int want_warps = kNumSMs * 32;
  int pool = 32;
  while (pool > 4 && (n + pool - 1) / pool < want_warps) pool >>= 1;
  return pool;
}

template <int VEC, int LPN, int NV, bool DEEP>
static int launch_spmm_impl(const int* rowptr, const int* col, const float* val, int n, int m, int64_t nnz, const float* B,
                       int64_t ldb64, float* C, int64_t ldc64, int f_eff, int f, float beta, const int* plan,
                       cudaStream_t stream) {
  const int ldb = static_cast<int>(ldb64), ldc = static_cast<int>(ldc64);   // checked to fit by the entry point
  (void)m;
  constexpr int TILE = LPN * VEC * NV;
  const int tiles = (f_eff + TILE - 1) / TILE;
  const int min_threshold = (LPN < 32) ? g_tuning.spmm_long_narrow : 0;
  if (plan) {
    // grid-stride over the listed rows, so any grid size is correct; this one is tight for the
    // current threshold and never below one wave
    const int blocks = max(1, min(plan_capacity(nnz, max(g_tuning.spmm_long, kMinLongThreshold)), 16 * kNumSMs));
    spmm_block_rows_kernel<VEC, LPN, NV, DEEP><<<dim3(blocks, tiles), kLongWarps * 32, 0, stream>>>(
        rowptr, col, val, B, ldb, C, ldc, f_eff, f, beta, plan, min_threshold);
  }
  const int rows_per_block = g_tuning.spmm_rpb;
  // the row kernel: allowed to start while the hub kernel's last rows are still running (see pdl_waiter_block)
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(rows_per_block * 32);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cfg.attrs = attr;
  // Measured on one box, serialised against overlapped: 4 M-vertex R-MAT graph width 128 7.99 -> 6.95 ms, width 602
  // 37.4 -> 36.8 ms; 233K-vertex graph width 602 with its dense core 10.14 -> 9.52 ms; width 16 0.78 -> 0.76 ms.
  cfg.numAttrs = (plan && g_tuning.spmm_overlap) ? 1 : 0;
  const int waiter = static_cast<int>(cfg.numAttrs);      // one block more, which only waits for the hub kernel
  cudaError_t e;
  bool grouped = false;
  if constexpr (LPN < 32) grouped = g_tuning.spmm_group_avg > 0 && nnz <= static_cast<int64_t>(g_tuning.spmm_group_avg) * n;
  if constexpr (LPN < 32) {
    if (grouped) {
      const int pool = group_pool_rows(n);
      const int pools = (n + pool - 1) / pool;
      cfg.gridDim = dim3((pools + rows_per_block - 1) / rows_per_block + waiter, tiles);
      e = cudaLaunchKernelEx(&cfg, spmm_group_rows_kernel<VEC, LPN, NV, DEEP>, rowptr, col, val, n, B, ldb, C, ldc, f_eff, f,
                             beta, plan, min_threshold, g_tuning.spmm_group_max, pool, waiter);
    }
  }
  if (!grouped) {
    cfg.gridDim = dim3((n + rows_per_block - 1) / rows_per_block + waiter, tiles);
    e = cudaLaunchKernelEx(&cfg, spmm_warp_rows_kernel<VEC, LPN, NV, DEEP>, rowptr, col, val, n, B, ldb, C, ldc, f_eff, f, beta,
                           plan, min_threshold, waiter);
  }
  if (e != cudaSuccess) {
    snprintf(last_error_buf(), 256, "cagnet_spmm_csr_f32: CUDA launch failed: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return CAGNET_E_LAUNCH;
  }
  return check_launch("cagnet_spmm_csr_f32");
}

template <int VEC, int LPN, int NV>
static int launch_spmm(const int* rowptr, const int* col, const float* val, int n, int m, int64_t nnz, const float* B,
                       int64_t ldb64, float* C, int64_t ldc64, int f_eff, int f, float beta, const int* plan,
                       cudaStream_t stream) {
  // Batched gathers pay where the multiply waits on memory latency with little else to run: one vector per lane
  // (at most 16 columns) on a block of short rows.  Measured on R-MAT graphs with 31 nonzeros per row: width 16
  // 0.585 -> 0.432 ms (1 M vertices), 2.09 -> 1.55 ms (4 M); but width 64 (two vectors per lane) 1.19 -> 1.30 ms, and
  // on a 233K-vertex graph with 493 nonzeros per row, where enough warps are resident to hide the latency and the
  // extra registers cost occupancy, width 16 0.80 -> 1.04 ms and width 41 1.62 -> 2.37 ms.
  if constexpr (LPN < 32 && NV == 1) {
    if (g_tuning.spmm_deep && g_tuning.spmm_group_avg > 0 && nnz <= static_cast<int64_t>(g_tuning.spmm_group_avg) * n)
      return launch_spmm_impl<VEC, LPN, NV, true>(rowptr, col, val, n, m, nnz, B, ldb64, C, ldc64, f_eff, f, beta, plan, stream);
  }
  return launch_spmm_impl<VEC, LPN, NV, false>(rowptr, col, val, n, m, nnz, B, ldb64, C, ldc64, f_eff, f, beta, plan, stream);
}

// Feature tiling.  A tile is `tile` vectors wide (tile * VEC columns); narrow B is covered by one tile of the
// next power of two.  Wide B is cut into 32-vector tiles (128 columns with 128-bit vectors): measured on a
// 233K-vertex / 115M-nonzero R-MAT graph at width 602, one 512-byte segment per gathered row and lane beat both
// narrower tiles (more passes over the col/val streams, more shuffles per byte) and the full-width tile (fewer
// resident warps, lower L1 hit rate on hub columns).
static int auto_tile(int vectors) {
  if (vectors <= 4) return 4;
  if (vectors <= 8) return 8;
  if (vectors <= 16) return 16;
  return 32;
}

template <int VEC>
static int dispatch_shape(int vectors, const int* rowptr, const int* col, const float* val, int n, int m, int64_t nnz,
                          const float* B, int64_t ldb, float* C, int64_t ldc, int f_eff, int f, float beta,
                          const int* plan, cudaStream_t stream) {
#define CAGNET_SPMM_CASE(LPN, NV) \
  return launch_spmm<VEC, LPN, NV>(rowptr, col, val, n, m, nnz, B, ldb, C, ldc, f_eff, f, beta, plan, stream)
  int tile = g_tuning.spmm_tile > 0 ? g_tuning.spmm_tile : auto_tile(vectors);
  if (vectors <= 4) tile = 4;
  if (g_tuning.spmm_tile == 0 && vectors > 4 && vectors <= 16) {
    // 5..16 vectors per row: two vectors per lane on a small lane group keep more lanes busy and more gathers in
    // flight than one power-of-two group (11 vectors on 16 lanes idle 5 of them).  Measured on the 233K-vertex /
    // 115M-nonzero graph: f = 41 1.69 ms against 2.54 ms, f = 64 1.75 against 2.56, f = 32 1.15 against 1.31.
    if (vectors <= 8) CAGNET_SPMM_CASE(4, 2);
    CAGNET_SPMM_CASE(8, 2);
  }
  switch (tile) {
    case 4: CAGNET_SPMM_CASE(4, 1);
    case 8: CAGNET_SPMM_CASE(8, 1);
    case 16: CAGNET_SPMM_CASE(16, 1);
    case 32: CAGNET_SPMM_CASE(32, 1);
    case 64: CAGNET_SPMM_CASE(32, 2);
    case 96: CAGNET_SPMM_CASE(32, 3);
    case 128: CAGNET_SPMM_CASE(32, 4);
    default: CAGNET_SPMM_CASE(32, 5);
  }
#undef CAGNET_SPMM_CASE
}

}  // namespace cagnet

using namespace cagnet;

extern "C" int cagnet_set_param(const char* name, int value) {
  if (!name) return fail(CAGNET_E_ARG, "cagnet_set_param: null name");
  if (!strcmp(name, "spmm_tile")) {
    const int ok[] = {0, 4, 8, 16, 32, 64, 96, 128, 160};
    for (int o : ok)
      if (value == o) {
        g_tuning.spmm_tile = value;
        return CAGNET_OK;
      }
    return fail(CAGNET_E_ARG, "cagnet_set_param: spmm_tile must be 0, 4, 8, 16, 32, 64, 96, 128 or 160");
  }
  if (!strcmp(name, "spmm_rpb")) {
    if (value != 1 && value != 2 && value != 4 && value != 8)
      return fail(CAGNET_E_ARG, "cagnet_set_param: spmm_rpb must be 1, 2, 4 or 8");
    g_tuning.spmm_rpb = value;
    return CAGNET_OK;
  }
  if (!strcmp(name, "core_chunk")) {
    if (set_core_chunk(value)) return fail(CAGNET_E_ARG, "cagnet_set_param: core_chunk must be a multiple of 32, >= 256");
    return CAGNET_OK;
  }
  if (!strcmp(name, "core_chunk_int")) {
    if (set_core_chunk_int(value)) return fail(CAGNET_E_ARG, "cagnet_set_param: core_chunk_int must be a multiple of 64, >= 256");
    return CAGNET_OK;
  }
  if (!strcmp(name, "spmm_long_narrow")) {
    if (value < kMinLongThreshold) return fail(CAGNET_E_ARG, "cagnet_set_param: spmm_long_narrow must be >= 256");
    g_tuning.spmm_long_narrow = value;
    return CAGNET_OK;
  }
  if (!strcmp(name, "spmm_group_max")) {
    if (value < 0 || value > 4096) return fail(CAGNET_E_ARG, "cagnet_set_param: spmm_group_max must be in [0, 4096]");
    g_tuning.spmm_group_max = value;
    return CAGNET_OK;
  }
  if (!strcmp(name, "spmm_group_pool")) {
    if (value != 0 && value != 4 && value != 8 && value != 16 && value != 32)
      return fail(CAGNET_E_ARG, "cagnet_set_param: spmm_group_pool must be 0, 4, 8, 16 or 32");
    g_tuning.spmm_group_pool = value;
    return CAGNET_OK;
  }
  if (!strcmp(name, "spmm_deep")) {
    g_tuning.spmm_deep = value != 0;
    return CAGNET_OK;
  }
  if (!strcmp(name, "spmm_overlap")) {
    g_tuning.spmm_overlap = value != 0;
    return CAGNET_OK;
  }
  if (!strcmp(name, "spmm_group_avg")) {
    if (value < 0) return fail(CAGNET_E_ARG, "cagnet_set_param: spmm_group_avg must be >= 0");
    g_tuning.spmm_group_avg = value;
    return CAGNET_OK;
  }
  if (!strcmp(name, "spmm_long")) {
    if (value < kMinLongThreshold) return fail(CAGNET_E_ARG, "cagnet_set_param: spmm_long must be >= 256");
    g_tuning.spmm_long = value;
    return CAGNET_OK;
  }
  return fail(CAGNET_E_ARG, "cagnet_set_param: unknown parameter '%s'", name);
}

extern "C" int cagnet_get_param(const char* name) {
  if (name && !strcmp(name, "spmm_tile")) return g_tuning.spmm_tile;
  if (name && !strcmp(name, "spmm_rpb")) return g_tuning.spmm_rpb;
  if (name && !strcmp(name, "spmm_long")) return g_tuning.spmm_long;
  if (name && !strcmp(name, "spmm_long_narrow")) return g_tuning.spmm_long_narrow;
  if (name && !strcmp(name, "spmm_group_max")) return g_tuning.spmm_group_max;
  if (name && !strcmp(name, "spmm_group_avg")) return g_tuning.spmm_group_avg;
  if (name && !strcmp(name, "spmm_group_pool")) return g_tuning.spmm_group_pool;
  if (name && !strcmp(name, "spmm_overlap")) return g_tuning.spmm_overlap;
  if (name && !strcmp(name, "spmm_deep")) return g_tuning.spmm_deep;
  if (name && !strcmp(name, "core_chunk")) return core_chunk();
  if (name && !strcmp(name, "core_chunk_int")) return core_chunk_int();
  return -1;
}

extern "C" size_t cagnet_spmm_plan_bytes(int32_t n, int64_t nnz) {
  (void)n;
  if (nnz < 0) return 0;
  return sizeof(int) * (kPlanHeaderInts + static_cast<size_t>(plan_capacity(nnz, kMinLongThreshold)));
}

extern "C" int cagnet_spmm_plan_i32(const int32_t* rowptr, int32_t n, int64_t nnz, void* plan, size_t plan_bytes,
                                    void* stream) {
  if (!rowptr || !plan || n < 0 || nnz < 0) return fail(CAGNET_E_ARG, "cagnet_spmm_plan_i32: bad argument");
  if (nnz > INT_MAX) return fail(CAGNET_E_OVERFLOW, "cagnet_spmm_plan_i32: nnz %s%lld exceeds int32", "", nnz);
  if (plan_bytes < cagnet_spmm_plan_bytes(n, nnz))
    return fail(CAGNET_E_WORKSPACE, "cagnet_spmm_plan_i32: plan buffer of %s%lld bytes is too small (need %lld)", "",
                (long long)plan_bytes, (long long)cagnet_spmm_plan_bytes(n, nnz));
  if (!aligned(plan, 16)) return fail(CAGNET_E_ALIGN, "cagnet_spmm_plan_i32: plan buffer must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threshold = g_tuning.spmm_long;
  const int capacity = plan_capacity(nnz, threshold);
  spmm_plan_header_kernel<<<1, 1, 0, s>>>(threshold, capacity, static_cast<int*>(plan));
  if (n > 0) launch_plan_passes(rowptr, n, threshold, capacity, static_cast<int*>(plan), s);
  return check_launch("cagnet_spmm_plan_i32");
}

// Argument checks shared by the two multiply entry points; `who` names the caller in the error text.
static int check_spmm_args(const char* who, const int32_t* rowptr, const int32_t* col, const float* val, int32_t n,
                           int32_t m, int64_t nnz, const float* B, int64_t ldb, float* C, int64_t ldc, int32_t f,
                           float beta) {
  if (n < 0 || m < 0 || nnz < 0 || f < 0) return fail(CAGNET_E_ARG, "%s: negative size", who);
  if (n == 0 || f == 0) return CAGNET_OK;
  if (!rowptr || !C || (nnz > 0 && (!col || !val || !B))) return fail(CAGNET_E_ARG, "%s: null pointer", who);
  if (beta != 0.f && beta != 1.f) return fail(CAGNET_E_ARG, "%s: beta must be 0 or 1", who);
  if (nnz > INT_MAX) return fail(CAGNET_E_OVERFLOW, "%s: nnz %lld exceeds int32", who, nnz);
  if (ldb < f || ldc < f)
    return fail(CAGNET_E_ALIGN, "%s: leading dimension (%lld, %lld) smaller than f", who, ldb, ldc);
  if (ldb > INT_MAX || ldc > INT_MAX)
    return fail(CAGNET_E_OVERFLOW, "%s: leading dimension (%lld, %lld) exceeds int32", who, ldb, ldc);
  return CAGNET_OK;
}

extern "C" int cagnet_spmm_csr_f32(const int32_t* rowptr, const int32_t* col, const float* val, int32_t n, int32_t m,
                                   int64_t nnz, const float* B, int64_t ldb, float* C, int64_t ldc, int32_t f,
                                   float beta, const void* plan, void* stream) {
  const int rc = check_spmm_args("cagnet_spmm_csr_f32", rowptr, col, val, n, m, nnz, B, ldb, C, ldc, f, beta);
  if (rc != CAGNET_OK || n == 0 || f == 0) return rc;
  if (!B) B = C;  // nnz == 0: never dereferenced
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int* p = static_cast<const int*>(plan);
  auto round_up = [](int x, int a) { return (x + a - 1) / a * a; };
  // Vector width by alignment.  Columns [f, round_up(f)) of B's padded rows are read (and their products thrown
  // away); C is only ever written below column f.
  if (ldb % 4 == 0 && ldc % 4 == 0 && aligned(B, 16) && aligned(C, 16) && round_up(f, 4) <= ldb && round_up(f, 4) <= ldc) {
    const int f_eff = round_up(f, 4);
    return dispatch_shape<4>(f_eff / 4, rowptr, col, val, n, m, nnz, B, ldb, C, ldc, f_eff, f, beta, p, s);
  }
  if (ldb % 2 == 0 && ldc % 2 == 0 && aligned(B, 8) && aligned(C, 8) && round_up(f, 2) <= ldb && round_up(f, 2) <= ldc) {
    const int f_eff = round_up(f, 2);
    return dispatch_shape<2>(f_eff / 2, rowptr, col, val, n, m, nnz, B, ldb, C, ldc, f_eff, f, beta, p, s);
  }
  return dispatch_shape<1>(f, rowptr, col, val, n, m, nnz, B, ldb, C, ldc, f, f, beta, p, s);
}

// ------------------------------------------------------------------------------------------------
// A multiply for callers that must not allocate.
//
// The ordinary entry point wants a plan buffer, which somebody has to allocate.  Some hosts cannot do that at
// the point of the call: a serving process whose device memory was handed, all of it, to another allocator at
// start-up (cudaMalloc then simply fails), or a latency-critical loop that may not take the implicit device
// synchronisation and driver lock that cudaMalloc/cudaFree bring with them.  For them the plan lives in the
// fixed device array below, which is part of the library image: every GPU that loads the library holds these
// 256 KB from load until exit whether or not the entry point is ever used.
namespace cagnet {

constexpr int kStaticPlanRows = 65536;   // at most this many hub rows can be listed
static __device__ __align__(256) int g_static_plan[kPlanHeaderInts + kStaticPlanRows];

// In host code `g_static_plan` is only a handle for the runtime, not a device address; the address has to be
// asked for, per device, with that device current.  Cached here after the first call on each device.
constexpr int kMaxDevices = 64;
static int* g_static_plan_addr[kMaxDevices] = {};

static int static_plan_address(int** out) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= kMaxDevices)
    return fail(CAGNET_E_LAUNCH, "cagnet_spmm_csr_f32_noalloc: cannot identify the current device%s (%lld)", "",
                static_cast<long long>(device));
  // concurrent first calls on one device all obtain the same address; the slot is read and written atomically
  if (!__atomic_load_n(&g_static_plan_addr[device], __ATOMIC_ACQUIRE)) {
    int* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_plan);
    if (e != cudaSuccess || !p) {
      snprintf(last_error_buf(), 256, "cagnet_spmm_csr_f32_noalloc: cudaGetSymbolAddress failed: %s",
               cudaGetErrorString(e));
      return CAGNET_E_LAUNCH;
    }
    __atomic_store_n(&g_static_plan_addr[device], p, __ATOMIC_RELEASE);
  }
  *out = __atomic_load_n(&g_static_plan_addr[device], __ATOMIC_ACQUIRE);
  return CAGNET_OK;
}

}  // namespace cagnet

extern "C" int64_t cagnet_spmm_noalloc_max_nnz(void) {
  // the hub-row list can never hold more than nnz / threshold + 1 rows, so this many nonzeros always fit
  return static_cast<int64_t>(kStaticPlanRows - 1) * g_tuning.spmm_long;
}

extern "C" int cagnet_spmm_csr_f32_noalloc(const int32_t* rowptr, const int32_t* col, const float* val, int32_t n,
                                           int32_t m, int64_t nnz, const float* B, int64_t ldb, float* C, int64_t ldc,
                                           int32_t f, float beta, void* stream) {
  // every argument is checked before anything is queued: a rejected call leaves the shared list as it was
  const int arc = check_spmm_args("cagnet_spmm_csr_f32_noalloc", rowptr, col, val, n, m, nnz, B, ldb, C, ldc, f, beta);
  if (arc != CAGNET_OK || n == 0 || f == 0) return arc;
  if (nnz > cagnet_spmm_noalloc_max_nnz())
    return fail(CAGNET_E_WORKSPACE,
                "cagnet_spmm_csr_f32_noalloc: %s%lld nonzeros exceed the built-in scratch (at most %lld at the current "
                "hub-row threshold); use cagnet_spmm_csr_f32 with a caller-allocated plan",
                "", nnz, static_cast<long long>(cagnet_spmm_noalloc_max_nnz()));
  int* plan = nullptr;
  const int rc = static_plan_address(&plan);
  if (rc != CAGNET_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threshold = g_tuning.spmm_long;
  const int capacity = min(plan_capacity(nnz, threshold), kStaticPlanRows);
  // the array keeps whatever the previous call left in it: the header kernel resets the row count first
  spmm_plan_header_kernel<<<1, 1, 0, s>>>(threshold, capacity, plan);
  launch_plan_passes(rowptr, n, threshold, capacity, plan, s);
  const int lrc = check_launch("cagnet_spmm_csr_f32_noalloc");
  if (lrc != CAGNET_OK) return lrc;
  return cagnet_spmm_csr_f32(rowptr, col, val, n, m, nnz, B, ldb, C, ldc, f, beta, plan, stream);
}
