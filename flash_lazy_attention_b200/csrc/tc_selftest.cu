// Self test of the tensor-core building blocks: one 128x128x128 bf16 tile product through
// TMA -> shared memory -> tcgen05.mma -> tensor memory -> registers, once per operand
// layout the attention kernels rely on.  No counterpart in the reference.
#include "common.cuh"
#include "tc_prims.cuh"

namespace fla {
namespace tc {

constexpr int ST_TILE_BYTES = 128 * 128 * 2;

__global__ void __launch_bounds__(128) selftest_kernel(const __grid_constant__ CUtensorMap map_a,
                                                       const __grid_constant__ CUtensorMap map_b,
                                                       const __nv_bfloat16* a_gmem, float* c, int variant,
                                                       int* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + ST_TILE_BYTES;
  __shared__ uint64_t bar_full, bar_mma;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar_full, 1);
    mbar_init(&bar_mma, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, 256);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  // variant 3: nothing is copied and nothing issued, so the first wait below runs out after a short
  // spin limit; the kernel then takes the same way out as the attention kernels after an expired
  // wait: error words written, every later wait returns at once, tensor memory freed, normal return.
  const uint32_t limit = variant == 3 ? (1u << 12) : kSpinLimit;
  if (tid == 0 && variant != 3) {
    mbar_expect_tx(&bar_full, 2 * ST_TILE_BYTES);
    tma_load_4d(sA, &map_a, &bar_full, 0, 0, 0, 0);
    tma_load_4d(sA + ST_TILE_BYTES / 2, &map_a, &bar_full, 64, 0, 0, 0);
    tma_load_4d(sB, &map_b, &bar_full, 0, 0, 0, 0);
    tma_load_4d(sB + ST_TILE_BYTES / 2, &map_b, &bar_full, 64, 0, 0, 0);
  }

  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  if (variant == 2) {
    // A operand into tensor-memory columns [128, 192): two bf16 per 32-bit column.
    const uint32_t* arow = (const uint32_t*)(a_gmem + (size_t)tid * 128);
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      uint32_t r[16];
#pragma unroll
      for (int x = 0; x < 16; ++x) {
        r[x] = arow[ch * 16 + x];
      }
      tmem_st16(tmem_base + lane_base + 128 + ch * 16, r);
    }
    tmem_st_wait();
  }
  mbar_wait(&bar_full, 0, &abort_flag, status, 1, limit);
  tc_fence_before_sync();
  __syncthreads();

  if (tid == 0 && variant != 3) {
    tc_fence_after_sync();
    const uint32_t a_addr = smem_u32(sA), b_addr = smem_u32(sB);
    if (variant == 0 || variant == 2) {
      const uint32_t idesc = make_idesc(128, 128, 1, 0, 0);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t off = (ks >> 2) * (ST_TILE_BYTES / 2) + (ks & 3) * 32;
        if (variant == 0) umma_ss(tmem_base, desc_kmajor(a_addr + off), desc_kmajor(b_addr + off), idesc, ks > 0);
        else umma_ts(tmem_base, tmem_base + 128 + ks * 8, desc_kmajor(b_addr + off), idesc, ks > 0);
      }
    } else {
      const uint32_t idesc = make_idesc(128, 128, 1, 0, 1);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t off = (ks >> 2) * (ST_TILE_BYTES / 2) + (ks & 3) * 32;
        umma_ss(tmem_base, desc_kmajor(a_addr + off), desc_mnmajor(b_addr + ks * 2048, ST_TILE_BYTES / 2), idesc,
                ks > 0);
      }
    }
    umma_commit(&bar_mma);
  }
  mbar_wait(&bar_mma, 0, &abort_flag, status, 2, limit);
  tc_fence_after_sync();
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    uint32_t r[32];
    tmem_ld32(tmem_base + lane_base + ch * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int x = 0; x < 32; ++x) c[(size_t)tid * 128 + ch * 32 + x] = variant == 3 ? 0.f : __uint_as_float(r[x]);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 256);
}

}  // namespace tc

cudaError_t selftest_umma_launch(const CUtensorMap& map_a, const CUtensorMap& map_b, const void* a, float* c,
                                 int variant, int* status, cudaStream_t st) {
  const size_t smem = 2 * tc::ST_TILE_BYTES + 1024;
  cudaError_t err =
      cudaFuncSetAttribute(tc::selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) return err;
  tc::selftest_kernel<<<1, 128, smem, st>>>(map_a, map_b, (const __nv_bfloat16*)a, c, variant, status);
  return cudaGetLastError();
}

}  // namespace fla
