// Rotary position embedding of q and k in one launch (rotate-half convention, angles in fp32).
//
// The step right before the attention operators in the reference's layers
// (examples/lazy_attention_layer.py:131, examples/sw_attention_lazy.py:150: RotaryEmbedding of q and k).  It is a
// separate, HBM-bound kernel and not part of the attention kernels' tile loads on purpose: a K tile is fetched by
// every query tile of its (batch, head) pair and once per pass over the keys -- several hundred times at the
// benchmark shapes -- so rotating at load time would repeat the rotation that often, in kernels whose row threads
// and shared-memory port are already the bound; rotating once costs one read and one write of q and k.
//
// Wide form (head dimension a multiple of 16, 16-byte aligned views; other even head dimensions and alignments take
// a scalar kernel).  One thread: 8 consecutive elements of the first half of a head row and the 8 partner elements of the second
// half (16-byte accesses for 16-bit types), for every head of one (batch, position): the sine and cosine of its 8
// angles are computed once and reused over the heads.  In place (out == in) is fine: a thread reads both halves
// before it writes them.
#include "common.cuh"

namespace fla {

namespace {

template <typename T>
struct Pack8;   // 8 elements
template <>
struct Pack8<float> {
  float4 a, b;
  __device__ void load(const float* p) { a = *(const float4*)p; b = *(const float4*)(p + 4); }
  __device__ void store(float* p) const { *(float4*)p = a; *(float4*)(p + 4) = b; }
  __device__ void get(float* f) const { f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w; }
  __device__ void set(const float* f) { a = make_float4(f[0], f[1], f[2], f[3]); b = make_float4(f[4], f[5], f[6], f[7]); }
};
template <typename T16>
struct Pack8_16 {
  uint4 w;
  __device__ void load(const T16* p) { w = *(const uint4*)p; }
  __device__ void store(T16* p) const { *(uint4*)p = w; }
  __device__ void get(float* f) const {
    const T16* e = reinterpret_cast<const T16*>(&w);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = to_f32<T16>(e[i]);
  }
  __device__ void set(const float* f) {
    T16* e = reinterpret_cast<T16*>(&w);
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = from_f32<T16>(f[i]);
  }
};
template <>
struct Pack8<__half> : Pack8_16<__half> {};
template <>
struct Pack8<__nv_bfloat16> : Pack8_16<__nv_bfloat16> {};

struct RopeTensor {
  const void* in;
  void* out;
  int64_t si[3], so[3];   // element strides of batch, head, position (inner stride 1)
  int H;
};

struct RopeParams {
  RopeTensor t[2];
  int B, L, D;
  float base;
  int offset;
  float sign;   // +1 rotate, -1 rotate back (the gradient of the rotation: it is orthogonal)
};

template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(const RopeParams p) {
  const int half = p.D >> 1;
  const int chunks = half >> 3;                       // 8-element chunks per half row
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int c = (int)(idx % chunks);
  const int64_t bl = idx / chunks;
  if (bl >= (int64_t)p.B * p.L) return;
  const int l = (int)(bl % p.L), b = (int)(bl / p.L);
  float cs[8], sn[8];
  const float pos = (float)(l + p.offset);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    // the same fp32 sequence as the dense formulation: inv = 1 / base^(j / half), angle = pos * inv
    const float inv = 1.0f / powf(p.base, (float)(c * 8 + i) / (float)half);
    sincosf(pos * inv, &sn[i], &cs[i]);
    sn[i] *= p.sign;
  }
#pragma unroll 1
  for (int t = 0; t < 2; ++t) {
    const RopeTensor& rt = p.t[t];
    if (rt.in == nullptr) continue;
#pragma unroll 2
    for (int h = 0; h < rt.H; ++h) {
      const T* src = (const T*)rt.in + (int64_t)b * rt.si[0] + (int64_t)h * rt.si[1] + (int64_t)l * rt.si[2] + c * 8;
      T* dst = (T*)rt.out + (int64_t)b * rt.so[0] + (int64_t)h * rt.so[1] + (int64_t)l * rt.so[2] + c * 8;
      Pack8<T> lo, hi;
      lo.load(src);
      hi.load(src + half);
      float x1[8], x2[8], y1[8], y2[8];
      lo.get(x1);
      hi.get(x2);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        y1[i] = x1[i] * cs[i] - x2[i] * sn[i];
        y2[i] = x2[i] * cs[i] + x1[i] * sn[i];
      }
      lo.set(y1);
      hi.set(y2);
      lo.store(dst);
      hi.store(dst + half);
    }
  }
}

// Any even head dimension, any alignment: one thread per (batch, position, frequency), scalar accesses.
template <typename T>
__global__ void __launch_bounds__(256) rope_kernel_scalar(const RopeParams p) {
  const int half = p.D >> 1;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int j = (int)(idx % half);
  const int64_t bl = idx / half;
  if (bl >= (int64_t)p.B * p.L) return;
  const int l = (int)(bl % p.L), b = (int)(bl / p.L);
  float cs, sn;
  sincosf((float)(l + p.offset) * (1.0f / powf(p.base, (float)j / (float)half)), &sn, &cs);
  sn *= p.sign;
  for (int t = 0; t < 2; ++t) {
    const RopeTensor& rt = p.t[t];
    if (rt.in == nullptr) continue;
    for (int h = 0; h < rt.H; ++h) {
      const T* src = (const T*)rt.in + (int64_t)b * rt.si[0] + (int64_t)h * rt.si[1] + (int64_t)l * rt.si[2] + j;
      T* dst = (T*)rt.out + (int64_t)b * rt.so[0] + (int64_t)h * rt.so[1] + (int64_t)l * rt.so[2] + j;
      const float x1 = to_f32<T>(src[0]), x2 = to_f32<T>(src[half]);
      dst[0] = from_f32<T>(x1 * cs - x2 * sn);
      dst[half] = from_f32<T>(x2 * cs + x1 * sn);
    }
  }
}

}  // namespace

cudaError_t rope_qk_launch(const View4* in, const View4* out, const int* heads, int B, int L, int D, float base,
                           int offset, int inverse, int dtype, cudaStream_t st) {
  RopeParams p;
  for (int t = 0; t < 2; ++t) {
    p.t[t].in = in[t].ptr;
    p.t[t].out = out[t].ptr;
    p.t[t].H = heads[t];
    p.t[t].si[0] = in[t].s[0]; p.t[t].si[1] = in[t].s[1]; p.t[t].si[2] = in[t].s[2];
    p.t[t].so[0] = out[t].s[0]; p.t[t].so[1] = out[t].s[1]; p.t[t].so[2] = out[t].s[2];
  }
  p.B = B; p.L = L; p.D = D; p.base = base; p.offset = offset; p.sign = inverse ? -1.f : 1.f;
  // 16-byte accesses need D a multiple of 16 and aligned bases and outer strides
  const int64_t unit = dtype == FLA_F32 ? 4 : 8;
  bool wide = D % 16 == 0;
  for (int t = 0; t < 2 && wide; ++t) {
    if (!in[t].ptr) continue;
    if ((((uintptr_t)in[t].ptr | (uintptr_t)out[t].ptr) & 15) != 0) wide = false;
    for (int i = 0; i < 3; ++i)
      if (in[t].s[i] % unit != 0 || out[t].s[i] % unit != 0) wide = false;
  }
  const int64_t threads = (int64_t)B * L * (wide ? D / 16 : D / 2);
  if (threads == 0) return cudaSuccess;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  if (wide) {
    if (dtype == FLA_F32) rope_kernel<float><<<grid, 256, 0, st>>>(p);
    else if (dtype == FLA_F16) rope_kernel<__half><<<grid, 256, 0, st>>>(p);
    else rope_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p);
  } else {
    if (dtype == FLA_F32) rope_kernel_scalar<float><<<grid, 256, 0, st>>>(p);
    else if (dtype == FLA_F16) rope_kernel_scalar<__half><<<grid, 256, 0, st>>>(p);
    else rope_kernel_scalar<__nv_bfloat16><<<grid, 256, 0, st>>>(p);
  }
  return cudaGetLastError();
}

}  // namespace fla
