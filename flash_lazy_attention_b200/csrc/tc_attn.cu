// Host side of the tensor-core (tcgen05 + TMEM + TMA) attention kernels: eligibility
// checks, tensor maps, template dispatch, launches.
#include "common.cuh"
#include "tc_bwd.cuh"
#include "tc_bwd_kv.cuh"
#include "tc_fwd.cuh"
#include "tc_prims.cuh"

namespace fla {

namespace {

// The tensor-core family takes bf16/fp16 tensors with D in {64, 128} whose rows can be fetched
// by TMA (unit inner stride, 16-byte aligned base and outer strides).
bool eligible(const AttnParams& p, int dtype, const char** why) {
  if (dtype != FLA_BF16 && dtype != FLA_F16) { *why = "tensor-core kernels take bf16 or fp16"; return false; }
  if (p.D != 64 && p.D != 128) { *why = "tensor-core kernels take head dim 64 or 128"; return false; }
  if ((int64_t)p.B * p.H * ((p.L + 127) / 128) > 0x7fffffffLL) { *why = "too many tiles"; return false; }
  if ((p.L + 63) / 64 > 32 * tc::kMaxMaskWords) { *why = "sequence too long for the block mask"; return false; }
  if ((p.L + 127) / 128 > tc::kBwdMaxTiles) { *why = "sequence too long for the backward tile list"; return false; }
  if (p.n_rep > 64 || (int64_t)p.n_rep * ((p.L + 127) / 128) > tc::kKvMaxTiles) {
    *why = "too many query heads per kv head for this sequence length";
    return false;
  }
  return true;
}

bool view_ok(const View4& v, const char** why) {
  if (!v.ptr) return true;
  if (((uintptr_t)v.ptr & 15) != 0) { *why = "a tensor base is not 16-byte aligned"; return false; }
  for (int i = 0; i < 3; ++i)
    if (v.s[i] < 0 || (v.s[i] & 7) != 0) { *why = "outer strides must be multiples of 8 elements"; return false; }
  return true;
}

template <int MODE, int D, bool LISTS, bool PAIR>
constexpr size_t fwd_smem_bytes() {   // the query tile(s), the K/V ring; with kept candidates: their staging slots
  return (size_t)tc::TileCfg<D>::kTileBytes * ((PAIR ? 2 : 1) + tc::TileCfg<D>::kStages) + 1024 +
         (PAIR ? 4 * tc::kMaxMaskWords : (MODE == ENTMAX ? tc::kStageBytes : 0));   // two-tile form: its second mask row
}

template <int MODE, int D, int FMT, int KIND, bool LISTS, bool PAIR = false>
cudaError_t launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnParams& p,
                       int* status, cudaStream_t st) {
  auto kern = tc::fwd_kernel<MODE, D, FMT, KIND, LISTS, PAIR>;
  constexpr size_t smem = fwd_smem_bytes<MODE, D, LISTS, PAIR>();
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int nmt = (p.L + 127) / 128;
  const unsigned grid = (unsigned)((PAIR ? (nmt + 1) / 2 : nmt) * p.B * p.H);
  kern<<<grid, tc::kFwdThreads, smem, st>>>(mq, mk, mv, p, status);
  return cudaGetLastError();
}

template <int MODE, int D, int FMT>
cudaError_t launch_fwd_kind(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnParams& p,
                            int* status, cudaStream_t st) {
  if constexpr (MODE == LAZY) {
    return launch_fwd<MODE, D, FMT, 0, false>(mq, mk, mv, p, status, st);
  } else {
    // Thresholds iterated on kept candidates or by passes over score tiles: alpha = 2 defaults to the
    // candidates, everything else to the passes (see the forward kernel); the flags override.
    const int kind = alpha_kind(p.alpha);
    const bool lists = (p.flags & FLA_FLAG_NO_CANDIDATE_LIST) ? false
                                                               : (kind == 1 || (p.flags & FLA_FLAG_CANDIDATE_LIST) != 0);
    // thresholds by score passes: two query tiles per CTA share every K tile they fetch (FLA_FLAG_ONE_TILE_CTAS
    // keeps the one-tile form)
    const bool pair = !lists && !(p.flags & FLA_FLAG_ONE_TILE_CTAS);
    if (pair) {
      switch (kind) {
        case 0: return launch_fwd<MODE, D, FMT, 0, false, true>(mq, mk, mv, p, status, st);
        case 1: return launch_fwd<MODE, D, FMT, 1, false, true>(mq, mk, mv, p, status, st);
        default: return launch_fwd<MODE, D, FMT, 2, false, true>(mq, mk, mv, p, status, st);
      }
    }
    switch (kind) {
      case 0: return lists ? launch_fwd<MODE, D, FMT, 0, true>(mq, mk, mv, p, status, st)
                           : launch_fwd<MODE, D, FMT, 0, false>(mq, mk, mv, p, status, st);
      case 1: return lists ? launch_fwd<MODE, D, FMT, 1, true>(mq, mk, mv, p, status, st)
                           : launch_fwd<MODE, D, FMT, 1, false>(mq, mk, mv, p, status, st);
      default: return lists ? launch_fwd<MODE, D, FMT, 2, true>(mq, mk, mv, p, status, st)
                            : launch_fwd<MODE, D, FMT, 2, false>(mq, mk, mv, p, status, st);
    }
  }
}

template <int MODE>
cudaError_t launch_fwd_shape(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnParams& p,
                             int dtype, int* status, cudaStream_t st) {
  const bool bf = dtype == FLA_BF16;
  if (p.D == 128) return bf ? launch_fwd_kind<MODE, 128, 1>(mq, mk, mv, p, status, st)
                            : launch_fwd_kind<MODE, 128, 0>(mq, mk, mv, p, status, st);
  return bf ? launch_fwd_kind<MODE, 64, 1>(mq, mk, mv, p, status, st)
            : launch_fwd_kind<MODE, 64, 0>(mq, mk, mv, p, status, st);
}

template <int MODE, int D>
constexpr size_t bwd_smem_bytes() {   // Q, dO, the K slots, two V slots
  return (size_t)tc::TileCfg<D>::kTileBytes * (4 + tc::kBwdKSlots) + 1024;
}

struct BwdMaps {
  CUtensorMap q, k, v, dout;   // 128-row boxes
};

template <int D>
constexpr size_t kv_smem_bytes() {   // K, V, two stages of (Q, dO)
  return (size_t)tc::TileCfg<D>::kTileBytes * (2 + 2 * tc::kKvStages) + 1024;
}

template <int MODE, int D, int FMT, int KIND>
cudaError_t launch_bwd(const BwdMaps& m, const AttnParams& p, int* status, cudaStream_t st) {
  const CUtensorMap &mq = m.q, &mk = m.k, &mv = m.v, &mdo = m.dout;
  auto kq = tc::dq_kernel<MODE, D, FMT, KIND>;
  auto kkv = tc::dkdv_kernel<MODE, D, FMT, KIND>;
  constexpr size_t smem = bwd_smem_bytes<MODE, D>();
  cudaError_t e = cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  constexpr size_t smem_kv = kv_smem_bytes<D>();
  e = cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv);
  if (e != cudaSuccess) return e;
  const unsigned grid = (unsigned)(((p.L + 127) / 128) * p.B * p.H);
  const unsigned grid_kv = (unsigned)(((p.L + 127) / 128) * p.B * p.Hkv);   // one CTA per key tile of a kv head
  // dq_kernel first: its first sweep produces the row scalars delta that dkdv_kernel reads
  // (development builds can leave out one of the two launches for timing experiments)
  kq<<<grid, tc::kBwdThreads, smem, st>>>(mq, mk, mv, mdo, p, status);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  kkv<<<grid_kv, tc::kKvThreads, smem_kv, st>>>(mq, mk, mv, mdo, p, status);
  return cudaGetLastError();
}

template <int MODE, int D, int FMT>
cudaError_t launch_bwd_kind(const BwdMaps& m, const AttnParams& p, int* status, cudaStream_t st) {
  if constexpr (MODE == LAZY) {
    return launch_bwd<MODE, D, FMT, 0>(m, p, status, st);
  } else {
    switch (alpha_kind(p.alpha)) {
      case 0: return launch_bwd<MODE, D, FMT, 0>(m, p, status, st);
      case 1: return launch_bwd<MODE, D, FMT, 1>(m, p, status, st);
      default: return launch_bwd<MODE, D, FMT, 2>(m, p, status, st);
    }
  }
}

template <int MODE>
cudaError_t launch_bwd_shape(const BwdMaps& m, const AttnParams& p, int dtype, int* status, cudaStream_t st) {
  const bool bf = dtype == FLA_BF16;
  if (p.D == 128) return bf ? launch_bwd_kind<MODE, 128, 1>(m, p, status, st)
                            : launch_bwd_kind<MODE, 128, 0>(m, p, status, st);
  return bf ? launch_bwd_kind<MODE, 64, 1>(m, p, status, st)
            : launch_bwd_kind<MODE, 64, 0>(m, p, status, st);
}

}  // namespace

// True when the tensor-core family will take a call with these q, k, v views (o, dO and the
// gradients are allocated by the caller to the same rules).
bool tc_attn_eligible(const AttnParams& p, int dtype, const char** why) {
  return eligible(p, dtype, why) && view_ok(p.q, why) && view_ok(p.k, why) && view_ok(p.v, why);
}

cudaError_t tc_attn_fwd(int mode, const AttnParams& p_in, int dtype, int* status, cudaStream_t st, const char** why) {
  AttnParams p = p_in;
  p.aux_o = nullptr;   // this family derives the backward's row scalars itself (dq_kernel, first sweep)
  p.aux_s = nullptr;
  if (!eligible(p, dtype, why)) return cudaErrorNotSupported;
  if (!view_ok(p.q, why) || !view_ok(p.k, why) || !view_ok(p.v, why) || !view_ok(p.o, why)) return cudaErrorNotSupported;
  CUtensorMap mq, mk, mv;
  if (!make_tensor_map_bhld(&mq, p.q.ptr, p.B, p.H, p.L, p.D, p.q.s, 128, why) ||
      !make_tensor_map_bhld(&mk, p.k.ptr, p.B, p.Hkv, p.L, p.D, p.k.s, 128, why) ||
      !make_tensor_map_bhld(&mv, p.v.ptr, p.B, p.Hkv, p.L, p.D, p.v.s, 128, why))
    return cudaErrorNotSupported;
  return mode == ENTMAX ? launch_fwd_shape<ENTMAX>(mq, mk, mv, p, dtype, status, st)
                        : launch_fwd_shape<LAZY>(mq, mk, mv, p, dtype, status, st);
}

cudaError_t tc_attn_bwd(int mode, const AttnParams& p, int dtype, int* status, cudaStream_t st, const char** why) {
  if (!eligible(p, dtype, why)) return cudaErrorNotSupported;
  if (!view_ok(p.q, why) || !view_ok(p.k, why) || !view_ok(p.v, why) || !view_ok(p.dout, why) ||
      !view_ok(p.dq, why) || !view_ok(p.dk, why) || !view_ok(p.dv, why))
    return cudaErrorNotSupported;
  BwdMaps m;
  if (!make_tensor_map_bhld(&m.q, p.q.ptr, p.B, p.H, p.L, p.D, p.q.s, 128, why) ||
      !make_tensor_map_bhld(&m.k, p.k.ptr, p.B, p.Hkv, p.L, p.D, p.k.s, 128, why) ||
      !make_tensor_map_bhld(&m.v, p.v.ptr, p.B, p.Hkv, p.L, p.D, p.v.s, 128, why) ||
      !make_tensor_map_bhld(&m.dout, p.dout.ptr, p.B, p.H, p.L, p.D, p.dout.s, 128, why))
    return cudaErrorNotSupported;
  return mode == ENTMAX ? launch_bwd_shape<ENTMAX>(m, p, dtype, status, st)
                        : launch_bwd_shape<LAZY>(m, p, dtype, status, st);
}

}  // namespace fla

