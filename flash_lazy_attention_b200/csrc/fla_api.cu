// extern "C" entry points of libflashlazy (declared in include/fla.h): argument
// validation, kernel-family selection, launches.  Nothing here allocates device memory,
// synchronises or changes the current device.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "tc_prims.cuh"

namespace fla {

// kernel families (defined in the other translation units)
cudaError_t simt_attn_fwd(int mode, const AttnParams& p, int dtype, cudaStream_t st);
cudaError_t simt_attn_bwd(int mode, const AttnParams& p, int dtype, cudaStream_t st);
cudaError_t attn_delta(int mode, const AttnParams& p, int dtype, cudaStream_t st);
cudaError_t entmax_rows_fwd(const void* x, void* y, int64_t rows, int64_t cols, float alpha, int n_iter, int fast,
                            int dtype, cudaStream_t st);
cudaError_t lazy_params_finish(const AttnParams& p, cudaStream_t st);
cudaError_t rope_qk_launch(const View4* in, const View4* out, const int* heads, int B, int L, int D, float base,
                           int offset, int inverse, int dtype, cudaStream_t st);
cudaError_t entmax_rows_bwd(const void* y, const void* dy, void* dx, int64_t rows, int64_t cols, float alpha,
                            int dtype, cudaStream_t st);
cudaError_t selftest_umma_launch(const CUtensorMap& map_a, const CUtensorMap& map_b, const void* a, float* c,
                                 int variant, int* status, cudaStream_t st);
// tensor-core family: returns cudaErrorNotSupported when it has no kernel for the request
cudaError_t tc_attn_fwd(int mode, const AttnParams& p, int dtype, int* status, cudaStream_t st, const char** why);
cudaError_t tc_attn_bwd(int mode, const AttnParams& p, int dtype, int* status, cudaStream_t st, const char** why);
bool tc_attn_eligible(const AttnParams& p, int dtype, const char** why);

static thread_local char g_err[512] = "";
static thread_local int g_last_path = 0;

static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
static int cuda_fail(cudaError_t e, const char* what) {
  return fail(FLA_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

// ---- tensor maps ----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

bool make_tensor_map_bhld(CUtensorMap* map, const void* ptr, int B, int H, int L, int D, const int64_t stride[4],
                          int box_rows, const char** err) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { *err = "cuTensorMapEncodeTiled is not available from the driver"; return false; }
  // The encoder is a driver entry point and needs the device's primary context bound to the
  // calling thread.  A thread that has only made cached allocations so far (an autograd worker)
  // may not have it yet; cudaFree(0) binds it without any other effect.
  static thread_local bool context_bound = false;
  if (!context_bound) { cudaFree(0); context_bound = true; }
  if (stride[3] != 1) { *err = "innermost stride must be 1"; return false; }
  if (((uintptr_t)ptr & 15) != 0) { *err = "base address must be 16-byte aligned"; return false; }
  for (int i = 0; i < 3; ++i)
    if (stride[i] < 0 || (stride[i] * 2) % 16 != 0) { *err = "strides must be non-negative multiples of 8 elements"; return false; }
  // the tiled encoding wants positive strides even for size-1 dimensions
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)L, (cuuint64_t)H, (cuuint64_t)B};
  int64_t sl = stride[2], sh = stride[1], sb = stride[0];
  if (sl == 0) sl = D;
  if (sh == 0) sh = (int64_t)L * sl;
  if (sb == 0) sb = (int64_t)H * sh;
  cuuint64_t strides[3] = {(cuuint64_t)sl * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64u, (cuuint32_t)box_rows, 1u, 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    static thread_local char msg[256];
    snprintf(msg, sizeof(msg),
             "cuTensorMapEncodeTiled rejected the view (code %d): dims %d,%d,%d,%d strides(elements) %lld,%lld,%lld ptr %p",
             (int)r, D, L, H, B, (long long)sl, (long long)sh, (long long)sb, ptr);
    *err = msg;
    return false;
  }
  return true;
}

// ---- validation helpers -----------------------------------------------------------------------
static int check_geom(const fla_attn_geom* g) {
  if (!g) return fail(FLA_ERR_INVALID, "geometry is NULL");
  if (g->B <= 0 || g->H <= 0 || g->L <= 0 || g->D <= 0)
    return fail(FLA_ERR_INVALID, "B, H, L, D must be positive (got %d %d %d %d)", g->B, g->H, g->L, g->D);
  if (g->dtype != FLA_F32 && g->dtype != FLA_F16 && g->dtype != FLA_BF16)
    return fail(FLA_ERR_INVALID, "unknown dtype %d", g->dtype);
  if (g->D > 128) return fail(FLA_ERR_UNSUPPORTED, "head dim %d > 128 is not supported", g->D);
  if (g->path < FLA_PATH_AUTO || g->path > FLA_PATH_TCGEN05) return fail(FLA_ERR_INVALID, "unknown path %d", g->path);
  if ((int64_t)g->B > 65535 || (int64_t)g->H > 65535) return fail(FLA_ERR_UNSUPPORTED, "B and H must be <= 65535");
  if (g->Hkv < 0 || (g->Hkv > 0 && (g->Hkv > g->H || g->H % g->Hkv != 0)))
    return fail(FLA_ERR_INVALID, "Hkv = %d must divide H = %d", g->Hkv, g->H);
  return FLA_OK;
}
static int check_view(const fla_tensor4* t, const char* name, View4* out) {
  if (!t || !t->ptr) return fail(FLA_ERR_INVALID, "tensor %s is NULL", name);
  if (t->stride[3] != 1) return fail(FLA_ERR_INVALID, "tensor %s: innermost stride must be 1 (got %lld)", name,
                                     (long long)t->stride[3]);
  out->ptr = t->ptr;
  for (int i = 0; i < 4; ++i) out->s[i] = t->stride[i];
  return FLA_OK;
}
#define FLA_TRY(expr) do { int _rc = (expr); if (_rc != FLA_OK) return _rc; } while (0)

static void fill_common(AttnParams& p, const fla_attn_geom* g) {
  memset(&p, 0, sizeof(p));
  p.B = g->B; p.H = g->H; p.L = g->L; p.D = g->D;
  p.Hkv = g->Hkv > 0 ? g->Hkv : g->H;
  p.n_rep = p.H / p.Hkv;
  p.causal = g->causal;
  p.varlen = g->varlen;
  p.scale = 1.0f / sqrtf((float)g->D);
  p.flags = g->flags;
}

// Runs `mode` forward or backward on the family the geometry selects.
static int dispatch(int mode, bool bwd, const fla_attn_geom* g, AttnParams& p, cudaStream_t st) {
  if (g->path != FLA_PATH_SIMT) {
    const char* why = "";
    cudaError_t e = bwd ? tc_attn_bwd(mode, p, g->dtype, g->status, st, &why)
                        : tc_attn_fwd(mode, p, g->dtype, g->status, st, &why);
    if (e == cudaSuccess) { g_last_path = FLA_PATH_TCGEN05; return FLA_OK; }
    if (e != cudaErrorNotSupported) return cuda_fail(e, "tensor-core launch");
    if (g->path == FLA_PATH_TCGEN05) return fail(FLA_ERR_UNSUPPORTED, "tensor-core path unavailable: %s", why);
  }
  if (p.n_rep != 1) return fail(FLA_ERR_UNSUPPORTED, "shared k/v heads (Hkv < H) need the tensor-core family");
  if (bwd) {
    if (!p.aux_o || (mode == ENTMAX && !p.aux_s))
      return fail(FLA_ERR_INVALID, "the SIMT family needs the aux buffers its forward filled");
    cudaError_t e = attn_delta(mode, p, g->dtype, st);
    if (e != cudaSuccess) return cuda_fail(e, "delta pre-pass launch");
  }
  cudaError_t e = bwd ? simt_attn_bwd(mode, p, g->dtype, st) : simt_attn_fwd(mode, p, g->dtype, st);
  if (e != cudaSuccess) return cuda_fail(e, "SIMT launch");
  g_last_path = FLA_PATH_SIMT;
  return FLA_OK;
}

}  // namespace fla

using namespace fla;

extern "C" {

int fla_version(void) { return 1100; }
const char* fla_last_error(void) { return g_err; }
int fla_last_path(void) { return g_last_path; }

int fla_device_supported(int device) {
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceProperties");
  if (prop.major != 10) return fail(FLA_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a",
                                    device, prop.major, prop.minor);
  return FLA_OK;
}

int fla_attn_uses_tensor_cores(const fla_attn_geom* g, const fla_tensor4* q, const fla_tensor4* k,
                               const fla_tensor4* v) {
  if (!g || !q || !k || !v || g->path == FLA_PATH_SIMT) return 0;
  if (g->B <= 0 || g->H <= 0 || g->L <= 0 || g->D <= 0) return 0;
  if (g->Hkv < 0 || (g->Hkv > 0 && (g->Hkv > g->H || g->H % g->Hkv != 0))) return 0;
  AttnParams p;
  fill_common(p, g);
  View4* dst[3] = {&p.q, &p.k, &p.v};
  const fla_tensor4* src[3] = {q, k, v};
  for (int t = 0; t < 3; ++t) {
    if (!src[t]->ptr || src[t]->stride[3] != 1) return 0;
    dst[t]->ptr = src[t]->ptr;
    for (int i = 0; i < 4; ++i) dst[t]->s[i] = src[t]->stride[i];
  }
  const char* why = "";
  return tc_attn_eligible(p, g->dtype, &why) ? 1 : 0;
}

int64_t fla_block_mask_words(int32_t L) { return ((int64_t)(L + 63) / 64 + 31) / 32; }

int fla_entmax_fwd(const void* x, void* y, int64_t rows, int64_t cols, float alpha, int n_iter, int fast_math,
                   int dtype, void* stream) {
  if (!x || !y) return fail(FLA_ERR_INVALID, "x or y is NULL");
  if (rows < 0 || cols <= 0 || cols > (1 << 30)) return fail(FLA_ERR_INVALID, "bad shape rows=%lld cols=%lld", (long long)rows, (long long)cols);
  if (!(alpha > 1.0f && alpha <= 2.0f)) return fail(FLA_ERR_INVALID, "alpha must be in (1, 2], got %g", alpha);
  if (n_iter < 0) return fail(FLA_ERR_INVALID, "n_iter must be >= 0");
  if (dtype < FLA_F32 || dtype > FLA_BF16) return fail(FLA_ERR_INVALID, "unknown dtype %d", dtype);
  if (rows == 0) return FLA_OK;
  cudaError_t e = entmax_rows_fwd(x, y, rows, cols, alpha, n_iter, fast_math, dtype, (cudaStream_t)stream);
  return e == cudaSuccess ? FLA_OK : cuda_fail(e, "entmax forward launch");
}

int fla_entmax_bwd(const void* y, const void* dy, void* dx, int64_t rows, int64_t cols, float alpha, int dtype,
                   void* stream) {
  if (!y || !dy || !dx) return fail(FLA_ERR_INVALID, "y, dy or dx is NULL");
  if (rows < 0 || cols <= 0 || cols > (1 << 30)) return fail(FLA_ERR_INVALID, "bad shape rows=%lld cols=%lld", (long long)rows, (long long)cols);
  if (!(alpha > 1.0f && alpha <= 2.0f)) return fail(FLA_ERR_INVALID, "alpha must be in (1, 2], got %g", alpha);
  if (dtype < FLA_F32 || dtype > FLA_BF16) return fail(FLA_ERR_INVALID, "unknown dtype %d", dtype);
  if (rows == 0) return FLA_OK;
  cudaError_t e = entmax_rows_bwd(y, dy, dx, rows, cols, alpha, dtype, (cudaStream_t)stream);
  return e == cudaSuccess ? FLA_OK : cuda_fail(e, "entmax backward launch");
}

int fla_rope_qk(const fla_tensor4* q_in, const fla_tensor4* q_out, int32_t Hq, const fla_tensor4* k_in,
                const fla_tensor4* k_out, int32_t Hk, int32_t B, int32_t L, int32_t D, int32_t dtype, float base,
                int32_t offset, int32_t inverse, void* stream) {
  if (!q_in || !q_out || !q_in->ptr || !q_out->ptr) return fail(FLA_ERR_INVALID, "q_in or q_out is NULL");
  if ((k_in == nullptr) != (k_out == nullptr)) return fail(FLA_ERR_INVALID, "k_in and k_out must both be given or both be NULL");
  if (dtype < FLA_F32 || dtype > FLA_BF16) return fail(FLA_ERR_INVALID, "unknown dtype %d", dtype);
  if (B < 0 || L < 0 || Hq < 1 || (k_in && Hk < 1)) return fail(FLA_ERR_INVALID, "bad shape B=%d L=%d Hq=%d Hk=%d", B, L, Hq, Hk);
  if (D < 2 || D % 2 != 0) return fail(FLA_ERR_INVALID, "head dim %d: rotate-half needs an even head dimension", D);
  if (!(base > 0.f)) return fail(FLA_ERR_INVALID, "base must be positive");
  View4 in[2] = {}, out[2] = {};
  const fla_tensor4* src[4] = {q_in, q_out, k_in, k_out};
  for (int t = 0; t < 4; ++t) {
    if (!src[t]) continue;
    if (!src[t]->ptr) return fail(FLA_ERR_INVALID, "a tensor pointer is NULL");
    if (src[t]->stride[3] != 1) return fail(FLA_ERR_UNSUPPORTED, "the head dimension must have stride 1");
    View4& v = (t & 1) ? out[t >> 1] : in[t >> 1];
    v.ptr = src[t]->ptr;
    for (int i = 0; i < 4; ++i) v.s[i] = src[t]->stride[i];
  }
  const int heads[2] = {Hq, k_in ? Hk : 0};
  cudaError_t e = rope_qk_launch(in, out, heads, B, L, D, base, offset, inverse, dtype, (cudaStream_t)stream);
  return e == cudaSuccess ? FLA_OK : cuda_fail(e, "rotary embedding launch");
}

int fla_check_status(const int32_t* status, void* stream) {
  if (!status) return fail(FLA_ERR_INVALID, "status is NULL");
  int32_t host[4] = {0, 0, 0, 0};
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemcpyAsync(host, status, sizeof(host), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return cuda_fail(e, "reading the status words");
  if (host[0] != 0)
    return fail(FLA_ERR_DEVICE, "a bounded wait ran out in a tensor-core kernel (wait %d, block %d): results of that launch are not valid",
                host[1], host[2]);
  return FLA_OK;
}

int fla_entmax_attn_fwd(const fla_attn_geom* g, const fla_tensor4* q, const fla_tensor4* k, const fla_tensor4* v,
                        const fla_tensor4* o, float alpha, int niter, float* tau, float* aux_o, float* aux_s,
                        uint32_t* block_mask, void* stream) {
  FLA_TRY(check_geom(g));
  if (!(alpha > 1.0f && alpha <= 2.0f)) return fail(FLA_ERR_INVALID, "alpha must be in (1, 2], got %g", alpha);
  if (niter < 0) return fail(FLA_ERR_INVALID, "niter must be >= 0");
  if (!tau) return fail(FLA_ERR_INVALID, "tau buffer is NULL");
  if ((aux_o == nullptr) != (aux_s == nullptr)) return fail(FLA_ERR_INVALID, "aux_o and aux_s must both be given or both be NULL");
  AttnParams p;
  fill_common(p, g);
  FLA_TRY(check_view(q, "q", &p.q));
  FLA_TRY(check_view(k, "k", &p.k));
  FLA_TRY(check_view(v, "v", &p.v));
  FLA_TRY(check_view(o, "o", &p.o));
  p.alpha = alpha; p.niter = niter; p.tau = tau; p.aux_o = aux_o; p.aux_s = aux_s;
  p.block_mask = block_mask;
  p.mask_words = (int)fla_block_mask_words(g->L);
  cudaStream_t st = (cudaStream_t)stream;
  if (block_mask) {
    size_t bytes = (size_t)g->B * g->H * ((g->L + 127) / 128) * p.mask_words * sizeof(uint32_t);
    cudaError_t e = cudaMemsetAsync(block_mask, 0, bytes, st);
    if (e != cudaSuccess) return cuda_fail(e, "clearing the block mask");
  }
  return dispatch(ENTMAX, false, g, p, st);
}

size_t fla_entmax_attn_bwd_workspace(const fla_attn_geom* g) {
  if (!g || g->B <= 0 || g->H <= 0 || g->L <= 0) return 0;
  return (((size_t)g->B * g->H * g->L * sizeof(float)) + 255) & ~(size_t)255;
}

int fla_entmax_attn_bwd(const fla_attn_geom* g, const fla_tensor4* q, const fla_tensor4* k, const fla_tensor4* v,
                        const fla_tensor4* dout, float alpha, const float* tau, const float* aux_o,
                        const float* aux_s, const uint32_t* block_mask, const fla_tensor4* dq, const fla_tensor4* dk,
                        const fla_tensor4* dv, void* workspace, size_t workspace_bytes, void* stream) {
  FLA_TRY(check_geom(g));
  if (!(alpha > 1.0f && alpha <= 2.0f)) return fail(FLA_ERR_INVALID, "alpha must be in (1, 2], got %g", alpha);
  if (!tau) return fail(FLA_ERR_INVALID, "tau from the forward is required");
  if (!workspace || workspace_bytes < fla_entmax_attn_bwd_workspace(g))
    return fail(FLA_ERR_INVALID, "workspace too small: need %zu bytes, got %zu", fla_entmax_attn_bwd_workspace(g), workspace_bytes);
  if (((uintptr_t)workspace & 255) != 0) return fail(FLA_ERR_INVALID, "workspace must be 256-byte aligned");
  AttnParams p;
  fill_common(p, g);
  FLA_TRY(check_view(q, "q", &p.q));
  FLA_TRY(check_view(k, "k", &p.k));
  FLA_TRY(check_view(v, "v", &p.v));
  FLA_TRY(check_view(dout, "dout", &p.dout));
  FLA_TRY(check_view(dq, "dq", &p.dq));
  FLA_TRY(check_view(dk, "dk", &p.dk));
  FLA_TRY(check_view(dv, "dv", &p.dv));
  p.alpha = alpha;
  p.tau = const_cast<float*>(tau);
  p.aux_o = const_cast<float*>(aux_o);
  p.aux_s = const_cast<float*>(aux_s);
  p.block_mask = const_cast<uint32_t*>(block_mask);
  p.mask_words = (int)fla_block_mask_words(g->L);
  p.delta = (float*)workspace;
  return dispatch(ENTMAX, true, g, p, (cudaStream_t)stream);
}

// ---- backward of entmax attention for callers that cannot allocate ----------------------------
// The row scalars delta[B*H*L] normally live in a workspace the caller allocates.  Here they live
// in a fixed array inside the library image, so the call needs no allocation at all.
#define FLA_STATIC_SCRATCH_ROWS (1 << 20)
static __device__ __align__(256) float g_static_delta[FLA_STATIC_SCRATCH_ROWS];

// In host code `g_static_delta` is only a handle; the device address has to be asked for, once
// per device, with that device current.
static float* static_delta_ptr(int* rc) {
  constexpr int kMaxDevices = 64;
  static float* ptrs[kMaxDevices] = {};
  static std::mutex mu;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { *rc = cuda_fail(e, "cudaGetDevice"); return nullptr; }
  if (dev < 0 || dev >= kMaxDevices) { *rc = fail(FLA_ERR_UNSUPPORTED, "device index %d out of range", dev); return nullptr; }
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_static_delta);
    if (e != cudaSuccess) { *rc = cuda_fail(e, "cudaGetSymbolAddress(static scratch)"); return nullptr; }
    if (!ptr) { *rc = fail(FLA_ERR_CUDA, "cudaGetSymbolAddress(static scratch) returned a null address"); return nullptr; }
    ptrs[dev] = ptr;
  }
  *rc = FLA_OK;
  return ptrs[dev];
}

int64_t fla_entmax_attn_bwd_static_max_rows(void) { return FLA_STATIC_SCRATCH_ROWS; }

int fla_entmax_attn_bwd_static(const fla_attn_geom* g, const fla_tensor4* q, const fla_tensor4* k,
                               const fla_tensor4* v, const fla_tensor4* dout, float alpha, const float* tau,
                               const float* aux_o, const float* aux_s, const uint32_t* block_mask,
                               const fla_tensor4* dq, const fla_tensor4* dk, const fla_tensor4* dv, void* stream) {
  FLA_TRY(check_geom(g));
  if (!(alpha > 1.0f && alpha <= 2.0f)) return fail(FLA_ERR_INVALID, "alpha must be in (1, 2], got %g", alpha);
  if (!tau) return fail(FLA_ERR_INVALID, "tau from the forward is required");
  const int64_t rows = (int64_t)g->B * g->H * g->L;
  if (rows > FLA_STATIC_SCRATCH_ROWS)
    return fail(FLA_ERR_UNSUPPORTED,
                "B*H*L = %lld rows exceed the %d rows of built-in scratch; use fla_entmax_attn_bwd with a workspace",
                (long long)rows, FLA_STATIC_SCRATCH_ROWS);
  AttnParams p;
  fill_common(p, g);
  FLA_TRY(check_view(q, "q", &p.q));
  FLA_TRY(check_view(k, "k", &p.k));
  FLA_TRY(check_view(v, "v", &p.v));
  FLA_TRY(check_view(dout, "dout", &p.dout));
  FLA_TRY(check_view(dq, "dq", &p.dq));
  FLA_TRY(check_view(dk, "dk", &p.dk));
  FLA_TRY(check_view(dv, "dv", &p.dv));
  int rc = FLA_OK;
  float* scratch = static_delta_ptr(&rc);
  if (!scratch) return rc;
  p.alpha = alpha;
  p.tau = const_cast<float*>(tau);
  p.aux_o = const_cast<float*>(aux_o);
  p.aux_s = const_cast<float*>(aux_s);
  p.block_mask = const_cast<uint32_t*>(block_mask);
  p.mask_words = (int)fla_block_mask_words(g->L);
  p.delta = scratch;  // every row a kernel reads is written earlier in the same call: nothing to clear
  return dispatch(ENTMAX, true, g, p, (cudaStream_t)stream);
}

int fla_lazy_attn_fwd(const fla_attn_geom* g, const fla_tensor4* q, const fla_tensor4* k, const fla_tensor4* v,
                      const fla_tensor4* o, const float* bias, int64_t bias_stride, const float* tau, int32_t window,
                      float* lse, float* aux_o, void* stream) {
  FLA_TRY(check_geom(g));
  if (!bias || !tau || !lse) return fail(FLA_ERR_INVALID, "bias, tau or lse is NULL");
  if (window < 0) return fail(FLA_ERR_INVALID, "window must be >= 0");
  if (window > 0 && bias_stride < window) return fail(FLA_ERR_INVALID, "bias rows hold %lld columns, window is %d", (long long)bias_stride, window);
  AttnParams p;
  fill_common(p, g);
  p.causal = 1;
  FLA_TRY(check_view(q, "q", &p.q));
  FLA_TRY(check_view(k, "k", &p.k));
  FLA_TRY(check_view(v, "v", &p.v));
  FLA_TRY(check_view(o, "o", &p.o));
  p.bias = bias; p.bias_stride = bias_stride; p.tau_h = tau; p.window = window; p.lse = lse; p.aux_o = aux_o;
  return dispatch(LAZY, false, g, p, (cudaStream_t)stream);
}

// delta [B,H,L] floats, then the fixed-point accumulators of dbias [H, L] and dtau [H] (64-bit words)
size_t fla_lazy_attn_bwd_workspace(const fla_attn_geom* g) {
  const size_t rows = fla_entmax_attn_bwd_workspace(g);
  if (rows == 0) return 0;
  return rows + ((((size_t)g->H * ((size_t)g->L + 1)) * sizeof(unsigned long long) + 255) & ~(size_t)255);
}

int fla_lazy_attn_bwd(const fla_attn_geom* g, const fla_tensor4* q, const fla_tensor4* k, const fla_tensor4* v,
                      const fla_tensor4* o, const fla_tensor4* dout, const float* bias, int64_t bias_stride,
                      const float* tau, int32_t window, const float* lse, const float* aux_o, const fla_tensor4* dq,
                      const fla_tensor4* dk, const fla_tensor4* dv, float* dbias, int64_t dbias_stride, float* dtau,
                      void* workspace, size_t workspace_bytes, void* stream) {
  FLA_TRY(check_geom(g));
  if (!bias || !tau || !lse) return fail(FLA_ERR_INVALID, "bias, tau and lse are required");
  if (window < 0) return fail(FLA_ERR_INVALID, "window must be >= 0");
  if (dbias && dbias_stride < window) return fail(FLA_ERR_INVALID, "dbias rows hold %lld columns, window is %d", (long long)dbias_stride, window);
  if (!workspace || workspace_bytes < fla_lazy_attn_bwd_workspace(g))
    return fail(FLA_ERR_INVALID, "workspace too small: need %zu bytes, got %zu", fla_lazy_attn_bwd_workspace(g), workspace_bytes);
  if (((uintptr_t)workspace & 255) != 0) return fail(FLA_ERR_INVALID, "workspace must be 256-byte aligned");
  AttnParams p;
  fill_common(p, g);
  p.causal = 1;
  FLA_TRY(check_view(q, "q", &p.q));
  FLA_TRY(check_view(k, "k", &p.k));
  FLA_TRY(check_view(v, "v", &p.v));
  FLA_TRY(check_view(o, "o", &p.o));
  FLA_TRY(check_view(dout, "dout", &p.dout));
  FLA_TRY(check_view(dq, "dq", &p.dq));
  FLA_TRY(check_view(dk, "dk", &p.dk));
  FLA_TRY(check_view(dv, "dv", &p.dv));
  p.bias = bias; p.bias_stride = bias_stride; p.tau_h = tau; p.window = window;
  p.lse = const_cast<float*>(lse); p.aux_o = const_cast<float*>(aux_o);
  p.dbias = dbias; p.dbias_stride = dbias_stride; p.dtau = dtau;
  p.delta = (float*)workspace;
  cudaStream_t st = (cudaStream_t)stream;
  const bool params = dbias != nullptr || dtau != nullptr;
  if (params) {
    // order-independent sums: the kernels add into 64-bit fixed-point accumulators behind delta, cleared here,
    // and lazy_params_finish turns them into dbias / dtau (which it overwrites)
    unsigned long long* acc = (unsigned long long*)((char*)workspace + fla_entmax_attn_bwd_workspace(g));
    p.dbias_acc = dbias ? acc : nullptr;
    p.dbias_acc_stride = g->L;
    p.dtau_acc = dtau ? acc + (size_t)g->H * g->L : nullptr;
    cudaError_t e = cudaMemsetAsync(acc, 0, ((size_t)g->H * ((size_t)g->L + 1)) * sizeof(unsigned long long), st);
    if (e != cudaSuccess) return cuda_fail(e, "clearing the dbias / dtau accumulators");
  }
  const int rc = dispatch(LAZY, true, g, p, st);
  if (rc != FLA_OK || !params) return rc;
  cudaError_t e = lazy_params_finish(p, st);
  return e == cudaSuccess ? FLA_OK : cuda_fail(e, "dbias / dtau finish launch");
}

int fla_selftest_umma(const void* a, const void* b, float* c, int variant, int32_t* status, void* stream) {
  if (!a || !b || !c || !status) return fail(FLA_ERR_INVALID, "NULL argument");
  if (variant < 0 || variant > 3) return fail(FLA_ERR_INVALID, "variant must be 0, 1, 2 or 3");
  CUtensorMap ma, mb;
  const int64_t stride[4] = {128 * 128, 128 * 128, 128, 1};
  const char* err = "";
  if (!make_tensor_map_bhld(&ma, a, 1, 1, 128, 128, stride, 128, &err)) return fail(FLA_ERR_CUDA, "tensor map A: %s", err);
  if (!make_tensor_map_bhld(&mb, b, 1, 1, 128, 128, stride, 128, &err)) return fail(FLA_ERR_CUDA, "tensor map B: %s", err);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(status, 0, 4 * sizeof(int32_t), st);
  if (e != cudaSuccess) return cuda_fail(e, "clearing status");
  e = selftest_umma_launch(ma, mb, a, c, variant, status, st);
  return e == cudaSuccess ? FLA_OK : cuda_fail(e, "selftest launch");
}

}  // extern "C"
