// Stand-alone alpha-entmax over the last dimension of a contiguous [rows, cols] array,
// forward and backward.  Replaces adasplash.triton_entmax (source absent from the
// reference checkout; API README.md:26-35, behaviour tests/test_triton_entmax.py).
//
// HBM-bound: x is read once and y written once.  A row is kept in registers while the
// threshold is iterated (Halley for alpha <= 1.5, Newton above, both safeguarded by the
// bisection bracket [max-1, max-n^-(alpha-1)]), about 32 values per thread.  Rows made of
// whole 16-byte chunks take the vectorised kernels, whose owner grows with the row:
//   up to 512 values     4, 8 or 16 lanes of a warp (8, 4 or 2 rows per warp)
//   up to 1024           one warp
//   up to 8192           2, 4 or 8 warps (named barrier per row group / block barrier)
//   up to 65536          a thread-block cluster of 2, 4 or 8 blocks; partial sums cross the
//                        blocks through distributed shared memory, one cluster barrier each
//                        (fp32 forward rows of up to 16384 values: one block, 64 values per thread)
//   up to 131072         (forward) a cluster of 8 blocks with 64 values per thread
// Other shapes and longer rows take the scalar kernels, which re-read rows longer than
// 8192 from memory (L2) on every iteration.
#include <cooperative_groups.h>
#include <type_traits>
#include "common.cuh"
#include "tc_prims.cuh"

namespace fla {
namespace rows {

__device__ __forceinline__ float sqrt_approx(float x) {
  float r;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}


__device__ __forceinline__ float ld_any(const void* p, int dtype, int64_t i) {
  if (dtype == FLA_F32) return ((const float*)p)[i];
  if (dtype == FLA_F16) return __half2float(((const __half*)p)[i]);
  return __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void st_any(void* p, int dtype, int64_t i, float x) {
  if (dtype == FLA_F32) ((float*)p)[i] = x;
  else if (dtype == FLA_F16) ((__half*)p)[i] = __float2half_rn(x);
  else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(x);
}

struct Sum3 { float a, b, c; };

// Barrier among the GW warps that own one row: the whole block when GW == 8, a named barrier per
// row group otherwise (groups are aligned runs of GW warps; ids 1..4).
template <int GW>
__device__ __forceinline__ void group_barrier(int wg_first_warp) {
  if (GW == 8) __syncthreads();
  else asm volatile("bar.sync %0, %1;" ::"r"(1 + wg_first_warp / GW), "r"(GW * 32) : "memory");
}

// Reduce over the GW warps that own one row.  scratch: GW*3 floats per group.
template <int GW>
__device__ __forceinline__ Sum3 group_sum3(Sum3 v, float* scratch, int lane, int wg) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    v.a += __shfl_xor_sync(0xffffffffu, v.a, o);
    v.b += __shfl_xor_sync(0xffffffffu, v.b, o);
    v.c += __shfl_xor_sync(0xffffffffu, v.c, o);
  }
  if (GW == 1) return v;
  __syncthreads();
  if (lane == 0) { scratch[wg * 3] = v.a; scratch[wg * 3 + 1] = v.b; scratch[wg * 3 + 2] = v.c; }
  __syncthreads();
  Sum3 r = {0.f, 0.f, 0.f};
#pragma unroll
  for (int w = 0; w < GW; ++w) { r.a += scratch[w * 3]; r.b += scratch[w * 3 + 1]; r.c += scratch[w * 3 + 2]; }
  return r;
}
// The same with one barrier: callers alternate `half` (0/1) between consecutive reductions, so the
// warps that are still reading one half never meet the writes of the next reduction.
// scratch: 2 * GW * 3 floats.
template <int GW, int LPR = 32>
__device__ __forceinline__ float group_max_g(float v, float* scratch, int lane, int wg, int first_warp) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if (GW == 1) return v;
  if (lane == 0) scratch[wg] = v;
  group_barrier<GW>(first_warp);
  float r = -INFINITY;
#pragma unroll
  for (int w = 0; w < GW; ++w) r = fmaxf(r, scratch[w]);
  return r;
}
template <int GW, int LPR = 32>
__device__ __forceinline__ Sum3 group_sum3_alt(Sum3 v, float* scratch, int lane, int wg, int half, int first_warp) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) {
    v.a += __shfl_xor_sync(0xffffffffu, v.a, o);
    v.b += __shfl_xor_sync(0xffffffffu, v.b, o);
    v.c += __shfl_xor_sync(0xffffffffu, v.c, o);
  }
  if (GW == 1) return v;
  float* sc = scratch + half * GW * 3;
  if (lane == 0) { sc[wg * 3] = v.a; sc[wg * 3 + 1] = v.b; sc[wg * 3 + 2] = v.c; }
  group_barrier<GW>(first_warp);
  Sum3 r = {0.f, 0.f, 0.f};
#pragma unroll
  for (int w = 0; w < GW; ++w) { r.a += sc[w * 3]; r.b += sc[w * 3 + 1]; r.c += sc[w * 3 + 2]; }
  return r;
}
template <int GW>
__device__ __forceinline__ float group_max(float v, float* scratch, int lane, int wg) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if (GW == 1) return v;
  __syncthreads();
  if (lane == 0) scratch[wg] = v;
  __syncthreads();
  float r = -INFINITY;
#pragma unroll
  for (int w = 0; w < GW; ++w) r = fmaxf(r, scratch[w]);
  return r;
}

template <int KIND>
__device__ __forceinline__ void accum(float d, float e, bool fast, Sum3& s) {
  if (d > 0.f) {
    float pw, u;
    if (KIND == 2 && !fast) { pw = powf(d, e); u = powf(d, e - 1.f); }
    else p_and_u<KIND>(d, e, pw, u);
    s.a += pw;
    s.b += u;
    s.c += (KIND == 0) ? 1.f : ((KIND == 1) ? 0.f : u / d);
  }
}

// ITEMS > 0: the row is held in registers (cols <= GW*32*ITEMS); ITEMS == 0: streamed.
template <int GW, int ITEMS, int KIND>
__global__ void __launch_bounds__(256) entmax_fwd_kernel(const void* x, void* y, int64_t rows, int cols,
                                                         float alpha, int n_iter, int fast, int dtype) {
  __shared__ float scratch[8 * 3];
  constexpr int GT = GW * 32;            // threads per row
  constexpr int RPB = 8 / GW;            // rows per block
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = warp / GW, wg = warp % GW;
  const int t = wg * 32 + lane;
  int64_t row = (int64_t)blockIdx.x * RPB + grp;
  const bool row_ok = row < rows;
  if (!row_ok) row = rows - 1;           // keep every thread in the block-wide barriers
  const int64_t base = row * cols;
  float* sc = scratch + (GW == 1 ? 0 : 0);
  const float am1 = alpha - 1.f, e = 1.f / am1;

  float v[ITEMS > 0 ? ITEMS : 1];
  float m = -INFINITY;
  if (ITEMS > 0) {
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      int c = t + k * GT;
      v[k] = c < cols ? ld_any(x, dtype, base + c) * am1 : -INFINITY;
      m = fmaxf(m, v[k]);
    }
  } else {
    for (int c = t; c < cols; c += GT) m = fmaxf(m, ld_any(x, dtype, base + c) * am1);
  }
  m = group_max<GW>(m, sc, lane, wg);

  float lo = -1.f, hi = -exp2f(-am1 * log2f((float)cols)), ts = -1.f;
  bool done = cols <= 1;
  for (int it = 0; it < n_iter; ++it) {
    Sum3 s = {0.f, 0.f, 0.f};
    if (ITEMS > 0) {
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) accum<KIND>((v[k] - m) - ts, e, fast != 0, s);
    } else {
      for (int c = t; c < cols; c += GT) accum<KIND>((ld_any(x, dtype, base + c) * am1 - m) - ts, e, fast != 0, s);
    }
    s = group_sum3<GW>(s, sc, lane, wg);
    if (!done) {
      float tn = tau_update(ts, s.a, s.b, s.c, e, lo, hi);
      if (fabsf(tn - ts) <= 1.2e-7f) done = true;
      ts = tn;
    }
    // `done` is uniform inside a row group; with GW == 8 the group is the block
    if (GW == 1 ? __all_sync(0xffffffffu, done) : done) break;
  }
  if (!row_ok) return;
  if (ITEMS > 0) {
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      int c = t + k * GT;
      if (c < cols) {
        float d = (v[k] - m) - ts;
        float pw = 0.f;
        if (d > 0.f) pw = (KIND == 2 && !fast) ? powf(d, e) : pow_e<KIND>(d, e);
        st_any(y, dtype, base + c, pw);
      }
    }
  } else {
    for (int c = t; c < cols; c += GT) {
      float d = (ld_any(x, dtype, base + c) * am1 - m) - ts;
      float pw = 0.f;
      if (d > 0.f) pw = (KIND == 2 && !fast) ? powf(d, e) : pow_e<KIND>(d, e);
      st_any(y, dtype, base + c, pw);
    }
  }
}

// dx = U (dy - sum(U dy)/sum(U)),  U = y^(2-alpha) where y > 0
template <int GW>
__global__ void __launch_bounds__(256) entmax_bwd_kernel(const void* y, const void* dy, void* dx, int64_t rows,
                                                         int cols, float alpha, int dtype) {
  __shared__ float scratch[8 * 3];
  constexpr int GT = GW * 32, RPB = 8 / GW;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = warp / GW, wg = warp % GW;
  const int t = wg * 32 + lane;
  int64_t row = (int64_t)blockIdx.x * RPB + grp;
  const bool row_ok = row < rows;
  if (!row_ok) row = rows - 1;
  const int64_t base = row * cols;
  const float ex = 2.f - alpha;
  const int kind = alpha_kind(alpha);
  Sum3 s = {0.f, 0.f, 0.f};
  for (int c = t; c < cols; c += GT) {
    float p = ld_any(y, dtype, base + c);
    if (p > 0.f) {
      float u = kind == 0 ? sqrtf(p) : (kind == 1 ? 1.f : exp2f(ex * log2f(p)));
      s.a += u;
      s.b += u * ld_any(dy, dtype, base + c);
    }
  }
  s = group_sum3<GW>(s, scratch, lane, wg);
  if (!row_ok) return;
  const float q = s.a > 0.f ? s.b / s.a : 0.f;
  for (int c = t; c < cols; c += GT) {
    float p = ld_any(y, dtype, base + c);
    float g = 0.f;
    if (p > 0.f) {
      float u = kind == 0 ? sqrtf(p) : (kind == 1 ? 1.f : exp2f(ex * log2f(p)));
      g = u * (ld_any(dy, dtype, base + c) - q);
    }
    st_any(dx, dtype, base + c, g);
  }
}

// ---- 16-byte vectorised variants ---------------------------------------------------------------
// Used when a row is a whole number of 16-byte chunks and starts on a 16-byte boundary.  Thread t of
// the GW warps of a row owns chunks t, t + GT, ...: CH chunks of NV = 4 (fp32) or 8 (16-bit) values,
// held in registers while the threshold is iterated.  Loads and stores bypass L1 (streaming).
// Rows longer than one block's register tile are owned by a thread-block cluster of CS blocks: every
// block reduces its part, pushes the result into the slot with its rank in every block's shared
// memory (distributed shared memory), and after one cluster barrier all blocks add the CS slots in
// the same order, so that they take identical decisions.  Callers alternate `half` between
// consecutive reductions: a block may already push the next result while a slower one still reads.
template <int CS>
struct ClusterSlots { float v[2][CS][3]; };
// A block may only write into another block's shared memory once that block has started: every block
// of a cluster arrives at the cluster barrier as its first action and waits for the others just before
// its first remote store, so that the wait hides behind the row loads.
__device__ __forceinline__ void cluster_arrive_started() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_started() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int CS>
__device__ __forceinline__ Sum3 cluster_sum3(Sum3 v, ClusterSlots<CS>* slots, int half, unsigned rank) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  if (threadIdx.x < CS) {
    float* dst = cluster.map_shared_rank(&slots->v[half][rank][0], threadIdx.x);
    dst[0] = v.a; dst[1] = v.b; dst[2] = v.c;
  }
  cluster.sync();
  Sum3 r = {0.f, 0.f, 0.f};
#pragma unroll
  for (int w = 0; w < CS; ++w) { r.a += slots->v[half][w][0]; r.b += slots->v[half][w][1]; r.c += slots->v[half][w][2]; }
  return r;
}
template <int CS>
__device__ __forceinline__ float cluster_max(float v, ClusterSlots<CS>* slots, int half, unsigned rank) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  if (threadIdx.x < CS) *cluster.map_shared_rank(&slots->v[half][rank][0], threadIdx.x) = v;
  cluster.sync();
  float r = -INFINITY;
#pragma unroll
  for (int w = 0; w < CS; ++w) r = fmaxf(r, slots->v[half][w][0]);
  return r;
}

template <int DT> struct Vec;
template <> struct Vec<FLA_F32> {
  static constexpr int NV = 4;
  static __device__ __forceinline__ void load(const void* p, int64_t chunk, float* v) {
    const float4 q = __ldcs((const float4*)p + chunk);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
  static __device__ __forceinline__ void store(void* p, int64_t chunk, const float* v) {
    __stcs((float4*)p + chunk, make_float4(v[0], v[1], v[2], v[3]));
  }
};
template <> struct Vec<FLA_F16> {
  static constexpr int NV = 8;
  static __device__ __forceinline__ uint4 load_raw(const void* p, int64_t chunk) { return __ldcs((const uint4*)p + chunk); }
  static __device__ __forceinline__ void unpack(const uint4& q, float* v) {
    const __half2* h = (const __half2*)&q;
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void load(const void* p, int64_t chunk, float* v) { unpack(load_raw(p, chunk), v); }
  static __device__ __forceinline__ void store(void* p, int64_t chunk, const float* v) {
    uint4 q;
    __half2* h = (__half2*)&q;
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    __stcs((uint4*)p + chunk, q);
  }
};
template <> struct Vec<FLA_BF16> {
  static constexpr int NV = 8;
  static __device__ __forceinline__ uint4 load_raw(const void* p, int64_t chunk) { return __ldcs((const uint4*)p + chunk); }
  static __device__ __forceinline__ void unpack(const uint4& q, float* v) {
    const uint32_t* w = (const uint32_t*)&q;
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
  static __device__ __forceinline__ void load(const void* p, int64_t chunk, float* v) { unpack(load_raw(p, chunk), v); }
  static __device__ __forceinline__ void store(void* p, int64_t chunk, const float* v) {
    uint4 q;
    __nv_bfloat162* h = (__nv_bfloat162*)&q;
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    __stcs((uint4*)p + chunk, q);
  }
};

// LPR < 32 (GW == 1 only): short rows, 32 / LPR of them per warp, each on LPR adjacent lanes, so that a
// thread still holds about 32 values and the per-iteration reductions and threshold update are shared.
// CS > 1 (GW == 8 only): one row per cluster of CS blocks, launched with that cluster dimension.
template <int GW, int CH, int KIND, int DT, int LPR = 32, int CS = 1>
__global__ void __launch_bounds__(256, CH * Vec<DT>::NV <= 32 ? 4 : 2) entmax_fwd_vec_kernel(const void* x, void* y, int64_t rows, int cols,
                                                             float alpha, int n_iter, int fast) {
  static_assert(LPR == 32 || GW == 1, "rows that share a warp are owned by that warp alone");
  static_assert(CS == 1 || GW == 8, "a cluster owns one row, each of its blocks a part of it");
  __shared__ float scratch_all[2 * 8 * 3];   // per row group: two halves of GW*3 floats (see group_sum3_alt)
  __shared__ ClusterSlots<CS> cslots;
  if (CS > 1) cluster_arrive_started();
  float* scratch = scratch_all + (threadIdx.x >> 5) / GW * (2 * GW * 3);
  constexpr int NV = Vec<DT>::NV, GT = GW * LPR * CS, RW = 32 / LPR, RPB = 8 / GW * RW, N = CH * NV;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = warp / GW, wg = warp % GW;
  const unsigned crank = CS > 1 ? blockIdx.x % CS : 0u;   // rank in a one-dimensional cluster
  const int t = LPR == 32 ? (int)crank * GW * 32 + wg * 32 + lane : (lane & (LPR - 1));
  int64_t row = CS > 1 ? (int64_t)(blockIdx.x / CS) : (int64_t)blockIdx.x * RPB + grp * RW + lane / LPR;
  const bool row_ok = row < rows;
  if (!row_ok) row = rows - 1;           // keep every thread in the block-wide barriers
  const int nchunks = cols / NV;
  const int64_t base = row * nchunks;
  const float am1 = alpha - 1.f, e = 1.f / am1;

  float v[N];
  float m = -INFINITY;
#pragma unroll
  for (int k = 0; k < CH; ++k) {
    const int c = t + k * GT;
    if (c < nchunks) {
      Vec<DT>::load(x, base + c, v + k * NV);
      // alpha = 1.5 keeps the raw values and scales inside the fused multiply-add of every pass
#pragma unroll
      for (int i = 0; i < NV; ++i) { if (KIND != 0) v[k * NV + i] *= am1; m = fmaxf(m, v[k * NV + i]); }
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i) v[k * NV + i] = -INFINITY;
    }
  }
  m = group_max_g<GW, LPR>(m, scratch, lane, wg, warp - wg);
  if (CS > 1) { cluster_wait_started(); m = cluster_max<CS>(m, &cslots, 0, crank); }
  if (KIND == 0) m *= am1;

  float lo = -1.f, hi = -exp2f(-am1 * log2f((float)cols)), ts = -1.f;
  bool done = cols <= 1;
  for (int it = 0; it < n_iter; ++it) {
    Sum3 s = {0.f, 0.f, 0.f};
    const float noff = -(m + ts);
    if (KIND == 0) {
      // alpha = 1.5: d <= 1 on the whole bracket, so a saturating add gives max(d, 0) (0 for -inf)
      // sums kept as packed pairs: one instruction serves two values
      uint64_t s0 = tc::pack2(0.f, 0.f), s1 = s0, s2 = s0;
#pragma unroll
      for (int i = 0; i < N; i += 2) {
        const float e0 = __saturatef(fmaf(v[i], am1, noff)), e1 = __saturatef(fmaf(v[i + 1], am1, noff));
        const uint64_t ee = tc::pack2(e0, e1);
        s0 = tc::fma2(ee, ee, s0);
        s1 = tc::add2(s1, ee);
        s2 = tc::add2(s2, tc::pack2(e0 > 0.f ? 1.f : 0.f, e1 > 0.f ? 1.f : 0.f));
      }
      s.a = tc::sum2(s0); s.b = tc::sum2(s1); s.c = tc::sum2(s2);
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) accum<KIND>(v[i] + noff, e, fast != 0, s);
    }
    s = group_sum3_alt<GW, LPR>(s, scratch, lane, wg, (it + 1) & 1, warp - wg);   // (first half still holds the row maxima)
    if (CS > 1) s = cluster_sum3<CS>(s, &cslots, (it + 1) & 1, crank);
    if (!done) {
      bool regular;
      float tn = tau_update(ts, s.a, s.b, s.c, e, lo, hi, &regular);
      if (KIND == 0 && it == 0 && GW > 1) {   // long rows: tail-model first step (see gpd_first_step)
        const float jump = gpd_first_step(s.a, s.b, s.c);
        if (jump > 0.f && ts + jump > tn && ts + jump <= hi) { tn = ts + jump; regular = false; }
      }
      // the step after a regular Halley (Newton) step of length d is of order d^3 (d^2)
      const float tol = regular ? (e >= 2.f ? 3e-3f : 3e-4f) : 1.2e-7f;
      if (fabsf(tn - ts) <= tol) done = true;
      ts = tn;
    }
    if (GW == 1 ? __all_sync(0xffffffffu, done) : done) break;
  }
  if (!row_ok) return;
  const float noff = -(m + ts);
#pragma unroll
  for (int k = 0; k < CH; ++k) {
    const int c = t + k * GT;
    if (c < nchunks) {
      float o[NV];
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        if (KIND == 0) {
          const float d = __saturatef(fmaf(v[k * NV + i], am1, noff));
          o[i] = d * d;
        } else {
          const float d = v[k * NV + i] + noff;
          o[i] = d > 0.f ? ((KIND == 2 && !fast) ? powf(d, e) : pow_e<KIND>(d, e)) : 0.f;
        }
      }
      Vec<DT>::store(y, base + c, o);
    }
  }
}

// U = y^(2-alpha) on the support (alpha = 1.5: the approximate square root, relative error 2^-23, 0 at 0)
template <int K>
__device__ __forceinline__ float bwd_weight(float p, float ex) {
  if (K == 0) return sqrt_approx(fmaxf(p, 0.f));
  if (K == 1) return p > 0.f ? 1.f : 0.f;
  return p > 0.f ? exp2f(ex * log2f(p)) : 0.f;
}

// dx = U (dy - sum(U dy)/sum(U)),  U = y^(2-alpha) where y > 0; rows up to GW*32*CH*NV values in registers
template <int GW, int CH, int DT, int CS = 1, int LPR = 32>
__global__ void __launch_bounds__(256, Vec<DT>::NV == 8 ? 4 : 3) entmax_bwd_vec_kernel(const void* y, const void* dy, void* dx, int64_t rows,
                                                             int cols, float alpha) {
  static_assert(CS == 1 || GW == 8, "a cluster owns one row, each of its blocks a part of it");
  static_assert(LPR == 32 || (GW == 1 && CS == 1), "rows that share a warp are owned by that warp alone");
  __shared__ float scratch_all[2 * 8 * 3];
  __shared__ ClusterSlots<CS> cslots;
  if (CS > 1) cluster_arrive_started();
  float* scratch = scratch_all + (threadIdx.x >> 5) / GW * (2 * GW * 3);
  constexpr int NV = Vec<DT>::NV, GT = GW * LPR * CS, RW = 32 / LPR, RPB = 8 / GW * RW, N = CH * NV;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = warp / GW, wg = warp % GW;
  const unsigned crank = CS > 1 ? blockIdx.x % CS : 0u;
  const int t = LPR == 32 ? (int)crank * GW * 32 + wg * 32 + lane : (lane & (LPR - 1));
  int64_t row = CS > 1 ? (int64_t)(blockIdx.x / CS) : (int64_t)blockIdx.x * RPB + grp * RW + lane / LPR;
  const bool row_ok = row < rows;
  if (!row_ok) row = rows - 1;
  const int nchunks = cols / NV;
  const int64_t base = row * nchunks;
  const float ex = 2.f - alpha;
  const int kind = alpha_kind(alpha);
  Sum3 s = {0.f, 0.f, 0.f};
  if constexpr (NV == 8) {
    // 16-bit rows stay packed in registers (a quarter of the registers of the unpacked pair of arrays, so
    // that more blocks and more loads are in flight per SM); U is recomputed for the second pass
    uint4 yr[CH], gr[CH];
#pragma unroll
    for (int k = 0; k < CH; ++k) {
      const int c = t + k * GT;
      if (c < nchunks) {
        yr[k] = Vec<DT>::load_raw(y, base + c);
        gr[k] = Vec<DT>::load_raw(dy, base + c);
      } else {
        yr[k] = make_uint4(0u, 0u, 0u, 0u);
        gr[k] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    auto both_passes = [&](auto kind_c) {
      constexpr int K = decltype(kind_c)::value;
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        float a[NV], b[NV];
        Vec<DT>::unpack(yr[k], a);
        Vec<DT>::unpack(gr[k], b);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const float w = bwd_weight<K>(a[i], ex);
          s.a += w;
          s.b = fmaf(w, b[i], s.b);
        }
      }
      s = group_sum3_alt<GW, LPR>(s, scratch, lane, wg, 0, warp - wg);
      if (CS > 1) { cluster_wait_started(); s = cluster_sum3<CS>(s, &cslots, 0, crank); }
      if (!row_ok) return;
      const float q = s.a > 0.f ? s.b / s.a : 0.f;
      // (opaque to the compiler, which would otherwise keep the unpacked values of the first pass alive)
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        asm volatile("" : "+r"(yr[k].x), "+r"(yr[k].y), "+r"(yr[k].z), "+r"(yr[k].w));
        asm volatile("" : "+r"(gr[k].x), "+r"(gr[k].y), "+r"(gr[k].z), "+r"(gr[k].w));
      }
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        const int c = t + k * GT;
        if (c < nchunks) {
          float a[NV], b[NV], o[NV];
          Vec<DT>::unpack(yr[k], a);
          Vec<DT>::unpack(gr[k], b);
#pragma unroll
          for (int i = 0; i < NV; ++i) o[i] = bwd_weight<K>(a[i], ex) * (b[i] - q);
          Vec<DT>::store(dx, base + c, o);
        }
      }
    };
    if (kind == 0) both_passes(std::integral_constant<int, 0>{});
    else if (kind == 1) both_passes(std::integral_constant<int, 1>{});
    else both_passes(std::integral_constant<int, 2>{});
  } else {
    float u[N], g[N];
#pragma unroll
    for (int k = 0; k < CH; ++k) {
      const int c = t + k * GT;
      if (c < nchunks) {
        Vec<DT>::load(y, base + c, u + k * NV);
        Vec<DT>::load(dy, base + c, g + k * NV);
      } else {
#pragma unroll
        for (int i = 0; i < NV; ++i) { u[k * NV + i] = 0.f; g[k * NV + i] = 0.f; }
      }
    }
    // one loop per kind of alpha so that the common ones stay short
    auto weights = [&](auto kind_c) {
      constexpr int K = decltype(kind_c)::value;
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const float w = bwd_weight<K>(u[i], ex);
        u[i] = w;
        s.a += w;
        s.b = fmaf(w, g[i], s.b);
      }
    };
    if (kind == 0) weights(std::integral_constant<int, 0>{});
    else if (kind == 1) weights(std::integral_constant<int, 1>{});
    else weights(std::integral_constant<int, 2>{});
    s = group_sum3_alt<GW, LPR>(s, scratch, lane, wg, 0, warp - wg);
    if (CS > 1) { cluster_wait_started(); s = cluster_sum3<CS>(s, &cslots, 0, crank); }
    if (!row_ok) return;
    const float q = s.a > 0.f ? s.b / s.a : 0.f;
#pragma unroll
    for (int k = 0; k < CH; ++k) {
      const int c = t + k * GT;
      if (c < nchunks) {
        float o[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) o[i] = u[k * NV + i] * (g[k * NV + i] - q);
        Vec<DT>::store(dx, base + c, o);
      }
    }
  }
}

template <int GW, int CH, int DT, int LPR = 32>
static void launch_fwd_vec(const void* x, void* y, int64_t rows, int cols, float alpha, int n_iter, int fast,
                           cudaStream_t st) {
  constexpr int RPB = 8 / GW * (32 / LPR);
  const unsigned grid = (unsigned)((rows + RPB - 1) / RPB);
  const int kind = alpha_kind(alpha);
  if (kind == 0) entmax_fwd_vec_kernel<GW, CH, 0, DT, LPR><<<grid, 256, 0, st>>>(x, y, rows, cols, alpha, n_iter, fast);
  else if (kind == 1) entmax_fwd_vec_kernel<GW, CH, 1, DT, LPR><<<grid, 256, 0, st>>>(x, y, rows, cols, alpha, n_iter, fast);
  else entmax_fwd_vec_kernel<GW, CH, 2, DT, LPR><<<grid, 256, 0, st>>>(x, y, rows, cols, alpha, n_iter, fast);
}
// One row per cluster of CS blocks of 8 warps.
template <typename... Args>
static void launch_clustered(void (*kernel)(Args...), int cs, int64_t rows, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(rows * cs));
  cfg.blockDim = dim3(256);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, args...);
}
template <int CS, int CH, int DT>
static void launch_fwd_cluster(const void* x, void* y, int64_t rows, int cols, float alpha, int n_iter, int fast,
                               cudaStream_t st) {
  const int kind = alpha_kind(alpha);
  if (kind == 0) launch_clustered(entmax_fwd_vec_kernel<8, CH, 0, DT, 32, CS>, CS, rows, st, x, y, rows, cols, alpha, n_iter, fast);
  else if (kind == 1) launch_clustered(entmax_fwd_vec_kernel<8, CH, 1, DT, 32, CS>, CS, rows, st, x, y, rows, cols, alpha, n_iter, fast);
  else launch_clustered(entmax_fwd_vec_kernel<8, CH, 2, DT, 32, CS>, CS, rows, st, x, y, rows, cols, alpha, n_iter, fast);
}
// Picks the smallest register tile that holds a row; false if the row is too long.
template <int DT>
static bool launch_fwd_vec_dt(const void* x, void* y, int64_t rows, int cols, float alpha, int n_iter, int fast,
                              cudaStream_t st) {
  constexpr int NV = Vec<DT>::NV;
  const int chunks = cols / NV;
  // about 32 values per thread: 4, 8, 16 or 32 lanes per row up to 8 (fp32) / 4 (16-bit) chunks per
  // lane, then 2, 4, 8 warps per row; the longest register-resident rows take 64 values per thread
  constexpr int C = NV == 4 ? 8 : 4;     // chunks per thread for 32 values
  if (chunks <= 2 * C) launch_fwd_vec<1, C / 2, DT, 4>(x, y, rows, cols, alpha, n_iter, fast, st);
  else if (chunks <= 4 * C) launch_fwd_vec<1, C, DT, 4>(x, y, rows, cols, alpha, n_iter, fast, st);
  else if (chunks <= 8 * C) launch_fwd_vec<1, C, DT, 8>(x, y, rows, cols, alpha, n_iter, fast, st);
  else if (chunks <= 16 * C) launch_fwd_vec<1, C, DT, 16>(x, y, rows, cols, alpha, n_iter, fast, st);
  else if (chunks <= 32 * C) launch_fwd_vec<1, C, DT>(x, y, rows, cols, alpha, n_iter, fast, st);
  else if (chunks <= 64 * C) launch_fwd_vec<2, C, DT>(x, y, rows, cols, alpha, n_iter, fast, st);
  else if (chunks <= 128 * C) launch_fwd_vec<4, C, DT>(x, y, rows, cols, alpha, n_iter, fast, st);
  else if (chunks <= 256 * C) launch_fwd_vec<8, C, DT>(x, y, rows, cols, alpha, n_iter, fast, st);
  // (fp32 rows of up to 16384 values are faster in one block with 64 values per thread)
  else if (NV == 4 && chunks <= 512 * C) launch_fwd_vec<8, 2 * C, DT>(x, y, rows, cols, alpha, n_iter, fast, st);
  else if (rows * 8 > 0x7fffffffLL) return false;
  // longer rows: clusters of 2, 4, 8 blocks, still about 32 values per thread (64 for the longest)
  else if (chunks <= 512 * C) launch_fwd_cluster<2, C, DT>(x, y, rows, cols, alpha, n_iter, fast, st);
  else if (chunks <= 1024 * C) launch_fwd_cluster<4, C, DT>(x, y, rows, cols, alpha, n_iter, fast, st);
  else if (chunks <= 2048 * C) launch_fwd_cluster<8, C, DT>(x, y, rows, cols, alpha, n_iter, fast, st);
  else if (chunks <= 4096 * C) launch_fwd_cluster<8, 2 * C, DT>(x, y, rows, cols, alpha, n_iter, fast, st);
  else return false;
  return true;
}
template <int DT>
static bool launch_bwd_vec_dt(const void* y, const void* dy, void* dx, int64_t rows, int cols, float alpha,
                              cudaStream_t st) {
  constexpr int NV = Vec<DT>::NV;
  const int chunks = cols / NV;
  constexpr int C = NV == 4 ? 8 : 4;
  auto grid = [&](int gw) { const int rpb = 8 / gw; return (unsigned)((rows + rpb - 1) / rpb); };
  auto grid_sub = [&](int lpr) { const int rpb = 8 * (32 / lpr); return (unsigned)((rows + rpb - 1) / rpb); };
  // short rows share a warp (4 chunks per lane), so that enough loads are in flight per thread
  if (chunks <= 16) entmax_bwd_vec_kernel<1, 4, DT, 1, 4><<<grid_sub(4), 256, 0, st>>>(y, dy, dx, rows, cols, alpha);
  else if (chunks <= 32) entmax_bwd_vec_kernel<1, 4, DT, 1, 8><<<grid_sub(8), 256, 0, st>>>(y, dy, dx, rows, cols, alpha);
  else if (chunks <= 64) entmax_bwd_vec_kernel<1, 4, DT, 1, 16><<<grid_sub(16), 256, 0, st>>>(y, dy, dx, rows, cols, alpha);
  else if (chunks <= 128) entmax_bwd_vec_kernel<1, 4, DT><<<grid(1), 256, 0, st>>>(y, dy, dx, rows, cols, alpha);
  else if (chunks <= 256) entmax_bwd_vec_kernel<8, 1, DT><<<grid(8), 256, 0, st>>>(y, dy, dx, rows, cols, alpha);
  else if (chunks <= 512) entmax_bwd_vec_kernel<8, 2, DT><<<grid(8), 256, 0, st>>>(y, dy, dx, rows, cols, alpha);
  else if (chunks <= 1024) entmax_bwd_vec_kernel<8, 4, DT><<<grid(8), 256, 0, st>>>(y, dy, dx, rows, cols, alpha);
  else if (chunks <= 256 * C) entmax_bwd_vec_kernel<8, C, DT><<<grid(8), 256, 0, st>>>(y, dy, dx, rows, cols, alpha);
  else if (rows * 8 > 0x7fffffffLL) return false;
  else if (chunks <= 512 * C) launch_clustered(entmax_bwd_vec_kernel<8, C, DT, 2>, 2, rows, st, y, dy, dx, rows, cols, alpha);
  else if (chunks <= 1024 * C) launch_clustered(entmax_bwd_vec_kernel<8, C, DT, 4>, 4, rows, st, y, dy, dx, rows, cols, alpha);
  else if (chunks <= 2048 * C) launch_clustered(entmax_bwd_vec_kernel<8, C, DT, 8>, 8, rows, st, y, dy, dx, rows, cols, alpha);
  else return false;
  return true;
}

template <int GW, int ITEMS>
static void launch_fwd_cfg(const void* x, void* y, int64_t rows, int cols, float alpha, int n_iter, int fast,
                           int dtype, cudaStream_t st) {
  constexpr int RPB = 8 / GW;
  unsigned grid = (unsigned)((rows + RPB - 1) / RPB);
  int kind = alpha_kind(alpha);
  if (kind == 0) entmax_fwd_kernel<GW, ITEMS, 0><<<grid, 256, 0, st>>>(x, y, rows, cols, alpha, n_iter, fast, dtype);
  else if (kind == 1) entmax_fwd_kernel<GW, ITEMS, 1><<<grid, 256, 0, st>>>(x, y, rows, cols, alpha, n_iter, fast, dtype);
  else entmax_fwd_kernel<GW, ITEMS, 2><<<grid, 256, 0, st>>>(x, y, rows, cols, alpha, n_iter, fast, dtype);
}

}  // namespace rows

cudaError_t entmax_rows_fwd(const void* x, void* y, int64_t rows, int64_t cols, float alpha, int n_iter,
                            int fast, int dtype, cudaStream_t st) {
  using namespace rows;
  int c = (int)cols;
  {
    const int esz = dtype == FLA_F32 ? 4 : 2, nv = 16 / esz;
    const bool aligned = c % nv == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0;
    bool launched = false;
    if (aligned && c > 32) {
      if (dtype == FLA_F32) launched = launch_fwd_vec_dt<FLA_F32>(x, y, rows, c, alpha, n_iter, fast, st);
      else if (dtype == FLA_F16) launched = launch_fwd_vec_dt<FLA_F16>(x, y, rows, c, alpha, n_iter, fast, st);
      else launched = launch_fwd_vec_dt<FLA_BF16>(x, y, rows, c, alpha, n_iter, fast, st);
    }
    if (launched) return cudaGetLastError();
  }
  if (c <= 32) launch_fwd_cfg<1, 1>(x, y, rows, c, alpha, n_iter, fast, dtype, st);
  else if (c <= 128) launch_fwd_cfg<1, 4>(x, y, rows, c, alpha, n_iter, fast, dtype, st);
  else if (c <= 512) launch_fwd_cfg<1, 16>(x, y, rows, c, alpha, n_iter, fast, dtype, st);
  else if (c <= 1024) launch_fwd_cfg<1, 32>(x, y, rows, c, alpha, n_iter, fast, dtype, st);
  else if (c <= 2048) launch_fwd_cfg<8, 8>(x, y, rows, c, alpha, n_iter, fast, dtype, st);
  else if (c <= 8192) launch_fwd_cfg<8, 32>(x, y, rows, c, alpha, n_iter, fast, dtype, st);
  else launch_fwd_cfg<8, 0>(x, y, rows, c, alpha, n_iter, fast, dtype, st);
  return cudaGetLastError();
}

cudaError_t entmax_rows_bwd(const void* y, const void* dy, void* dx, int64_t rows, int64_t cols, float alpha,
                            int dtype, cudaStream_t st) {
  using namespace rows;
  {
    const int esz = dtype == FLA_F32 ? 4 : 2, nv = 16 / esz;
    const bool aligned = cols % nv == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)dy & 15) == 0 && ((uintptr_t)dx & 15) == 0;
    bool launched = false;
    if (aligned && cols > 32) {
      if (dtype == FLA_F32) launched = launch_bwd_vec_dt<FLA_F32>(y, dy, dx, rows, (int)cols, alpha, st);
      else if (dtype == FLA_F16) launched = launch_bwd_vec_dt<FLA_F16>(y, dy, dx, rows, (int)cols, alpha, st);
      else launched = launch_bwd_vec_dt<FLA_BF16>(y, dy, dx, rows, (int)cols, alpha, st);
    }
    if (launched) return cudaGetLastError();
  }
  if (cols <= 1024) {
    unsigned grid = (unsigned)((rows + 7) / 8);
    entmax_bwd_kernel<1><<<grid, 256, 0, st>>>(y, dy, dx, rows, (int)cols, alpha, dtype);
  } else {
    entmax_bwd_kernel<8><<<(unsigned)rows, 256, 0, st>>>(y, dy, dx, rows, (int)cols, alpha, dtype);
  }
  return cudaGetLastError();
}

}  // namespace fla
