/*
 * C ABI of libflashlazy: hand-written sm_100a CUDA for the alpha-entmax / Lazy
 * Attention hot path.  This is the drop-in boundary: every entry point replaces
 * one host launcher (or absent upstream module) of the reference, cited per
 * declaration by the file:line inside the reference project.
 *
 * Conventions (all entry points):
 *   - return 0 (FLA_OK) or an FLA_ERR_* class; a human-readable message for the
 *     calling thread is available from fla_last_error();
 *   - nothing is thrown, no device memory is allocated, nothing synchronises the
 *     device, the current device is never changed: the caller owns every buffer
 *     (outputs, saved statistics, workspaces) and passes the cudaStream_t to
 *     enqueue on (as a void*; NULL is the legacy default stream).  Two documented
 *     exceptions: fla_entmax_attn_bwd_static keeps its scratch inside the library,
 *     and fla_check_status waits for the stream it is given;
 *   - all pointers are device pointers of the device that is current in the
 *     calling thread, except the POD descriptor structs, which are host memory;
 *   - attention tensors are [B,H,L,D] views described by element strides; the
 *     innermost stride must be 1;
 *   - invalid arguments are rejected before anything is launched.
 */
#ifndef FLA_H_
#define FLA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLA_OK 0
#define FLA_ERR_INVALID 1      /* bad shape / dtype / stride / NULL pointer            */
#define FLA_ERR_UNSUPPORTED 2  /* valid request this build has no kernel for           */
#define FLA_ERR_CUDA 3         /* a CUDA runtime / driver call failed                  */
#define FLA_ERR_DEVICE 4       /* a kernel reported a bounded wait that ran out        */

#define FLA_F32 0
#define FLA_F16 1
#define FLA_BF16 2

/* kernel family selection */
#define FLA_PATH_AUTO 0     /* tensor-core kernels when shape/dtype/strides allow, else SIMT */
#define FLA_PATH_SIMT 1     /* fp32 CUDA-core kernels: any dtype, any D <= 128               */
#define FLA_PATH_TCGEN05 2  /* tcgen05 + TMEM + TMA kernels: bf16/fp16, D in {64,128}        */

/* fla_attn_geom.flags (a sum of bits; 0 in normal use).  They change how the tensor-core
 * forward of entmax attention finds the row thresholds, not what it computes; tests use them to
 * reach every code path.                                                                       */
#define FLA_FLAG_NO_CANDIDATE_LIST 1  /* iterate the thresholds by passes over recomputed score  *
                                       * tiles instead of on the candidates kept by the first pass */
#define FLA_FLAG_PLAIN_FIRST_STEP 2   /* alpha = 1.5: plain Halley first step instead of the      *
                                       * tail-model step                                         */
#define FLA_FLAG_CANDIDATE_LIST 4     /* iterate the thresholds on kept candidates for every      *
                                       * alpha (the default does so for alpha = 2 only)          */
#define FLA_FLAG_ONE_TILE_CTAS 8      /* entmax forward by score passes: one query tile per      *
                                       * thread block (default: two, sharing every K tile fetch)  */

/* A strided [B,H,L,D] view; strides in elements, stride[3] must be 1. */
typedef struct fla_tensor4 {
  void* ptr;
  int64_t stride[4];
} fla_tensor4;

/* Problem geometry shared by the attention entry points. */
typedef struct fla_attn_geom {
  int32_t B, H, L, D;
  int32_t dtype;          /* FLA_F32 / FLA_F16 / FLA_BF16: type of q,k,v,o and their gradients */
  int32_t causal;         /* entmax attention only; Lazy Attention is always causal           */
  const int32_t* varlen;  /* device int32 [B]: valid leading tokens per sequence, or NULL      */
  int32_t path;           /* FLA_PATH_*                                                        */
  int32_t* status;        /* device int32[32], 8-byte aligned, or NULL.  Tensor-core kernels     *
                           * report here:                                                         *
                           * [0] != 0: a bounded wait ran out ([1] which wait, [2] which block); *
                           * [4],[5]: low/high word of a running count of 128x128xD tile         *
                           * products issued (the "executed FLOPs" figure); [6],[7]: forward     *
                           * CTAs that iterated the thresholds on kept candidates / by passes    *
                           * over score tiles; [8..19]: as 64-bit words, per kernel (forward, dQ,  *
                           * dK/dV) the bitwise complement of the earliest start and the latest   *
                           * end of its CTAs in nanoseconds of the GPU's global timer (0 = not    *
                           * set): the live per-kernel durations of the benchmark; [26..31]: as   *
                           * 64-bit words, per kernel the sum of its CTAs' lifetimes in the same   *
                           * nanoseconds (divided by SMs x duration: the share of the launch the   *
                           * SMs were occupied).  Never cleared by the library; the caller zeroes  *
                           * it.                                                                   */
  int32_t flags;          /* FLA_FLAG_*                                                         */
  int32_t Hkv;            /* grouped-query attention: k, v, dk, dv are [B,Hkv,L,D] views and query  *
                           * head h uses head h / (H / Hkv) of them; 0 or H: every query head its  *
                           * own (the reference materialises the repeat: repeat_kv,                *
                           * examples/sw_attention_lazy.py:30-41,154-157).  Tensor-core family only. */
} fla_attn_geom;

/* Library / ABI version (major*1000 + minor). */
int fla_version(void);

/* Message of the last error raised on the calling thread ("" if none). */
const char* fla_last_error(void);

/* 0 when `device` is a compute-capability 10.x GPU this library has code for. */
int fla_device_supported(int device);

/* Waits for `stream` and reads the status words a tensor-core kernel reports into
 * (fla_attn_geom.status, device int32[32]).  Returns FLA_ERR_DEVICE, with the wait and the block
 * in fla_last_error(), if a bounded wait of a kernel ran out since the words were last cleared:
 * the results of that launch are not valid.  FLA_OK otherwise.  The only entry point that
 * synchronises; callers that never call it pay nothing.                                       */
int fla_check_status(const int32_t* status, void* stream);

/* Which kernel family the last attention call of the calling thread used (FLA_PATH_*). */
int fla_last_path(void);

/* 1 when a call with this geometry and these q, k, v views runs on the tensor-core family
 * (given outputs / gradients that are 16-byte aligned with strides that are multiples of 8
 * elements), else 0.  The tensor-core family needs no aux buffers (see below).             */
int fla_attn_uses_tensor_cores(const fla_attn_geom* g, const fla_tensor4* q, const fla_tensor4* k,
                               const fla_tensor4* v);

/* ---- stand-alone alpha-entmax over the last dimension ------------------------------------
 * Replaces adasplash.triton_entmax.triton_entmax (source absent from the reference checkout;
 * API README.md:26-35, call form tests/test_triton_entmax.py:27,41).
 * x, y: contiguous [rows, cols].  n_iter caps the Halley/Newton iterations on tau.       */
int fla_entmax_fwd(const void* x, void* y, int64_t rows, int64_t cols, float alpha,
                   int n_iter, int fast_math, int dtype, void* stream);
/* dx = U * (dy - sum(U dy)/sum(U)), U = y^(2-alpha) on the support of y. */
int fla_entmax_bwd(const void* y, const void* dy, void* dx, int64_t rows, int64_t cols,
                   float alpha, int dtype, void* stream);

/* ---- alpha-entmax attention ---------------------------------------------------------------
 * Replaces adasplash.adasplash / adasplash.adasplash_no_block_mask (sources absent from the
 * reference checkout; API README.md:37-57, behaviour tests/test_adasplash.py:22-190).
 *
 * Block mask: bit (I, J) of block_mask says that query block I (128 rows) has a non-zero
 * probability in key block J (64 keys).  Layout uint32 [B,H,Tr,mask_words],
 * Tr = ceil(L/128), mask_words = ceil(ceil(L/64)/32); bit J%32 of word J/32.
 * NULL selects the variant without a mask.                                               */
int64_t fla_block_mask_words(int32_t L);

/* Forward.  tau: float [B,H,L], the row thresholds in (alpha-1)*score units (saved for the
 * backward).  aux_o (float [B,H,L,D]) and aux_s (float [B,H,L]) receive U.V and sum(U),
 * U = P^(2-alpha), when the SIMT family runs; the tensor-core family ignores them (its
 * backward recomputes the row scalars).  Pass both NULL when no backward will follow or when
 * fla_attn_uses_tensor_cores() says 1.                                                    */
int fla_entmax_attn_fwd(const fla_attn_geom* g, const fla_tensor4* q, const fla_tensor4* k,
                        const fla_tensor4* v, const fla_tensor4* o, float alpha, int niter,
                        float* tau, float* aux_o, float* aux_s, uint32_t* block_mask,
                        void* stream);


/* Bytes of caller-provided scratch the backward needs for this geometry. */
size_t fla_entmax_attn_bwd_workspace(const fla_attn_geom* g);

/* Backward.  block_mask may be NULL (every block visited).  workspace: device memory of
 * at least fla_entmax_attn_bwd_workspace(g) bytes, 256-byte aligned.                      */
int fla_entmax_attn_bwd(const fla_attn_geom* g, const fla_tensor4* q, const fla_tensor4* k,
                        const fla_tensor4* v, const fla_tensor4* dout, float alpha,
                        const float* tau, const float* aux_o, const float* aux_s,
                        const uint32_t* block_mask, const fla_tensor4* dq,
                        const fla_tensor4* dk, const fla_tensor4* dv, void* workspace,
                        size_t workspace_bytes, void* stream);

/* Backward without any allocation.  No counterpart in the reference.
 * Some callers cannot provide the workspace fla_entmax_attn_bwd asks for: code that runs where
 * device allocation is forbidden or unavailable -- inside a region where the framework's
 * allocator must not be re-entered, in a process whose memory pool is fixed up front, or from a
 * thin language binding that can pass pointers but has no allocator of its own.  This variant
 * keeps the per-row scratch (one float per query row, B*H*L of them) in an array built into the
 * library image instead, and calls no allocating routine.
 *   - Limit: B*H*L <= fla_entmax_attn_bwd_static_max_rows() (1,048,576 rows = 4 MiB, held by every
 *     GPU that loads the library until the process exits); larger problems are rejected with
 *     FLA_ERR_UNSUPPORTED and must use fla_entmax_attn_bwd.
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call before any stream capture begins.
 *   - All calls on a device share the one array and it keeps the last call's contents.  Nothing
 *     needs clearing (each call writes every entry it later reads), but two calls that overlap
 *     on the GPU (different streams) race on it: serialise them.
 * Arguments as fla_entmax_attn_bwd, without the workspace.                                     */
int64_t fla_entmax_attn_bwd_static_max_rows(void);
int fla_entmax_attn_bwd_static(const fla_attn_geom* g, const fla_tensor4* q, const fla_tensor4* k,
                               const fla_tensor4* v, const fla_tensor4* dout, float alpha,
                               const float* tau, const float* aux_o, const float* aux_s,
                               const uint32_t* block_mask, const fla_tensor4* dq,
                               const fla_tensor4* dk, const fla_tensor4* dv, void* stream);

/* ---- Lazy Attention -------------------------------------------------------------------------
 * fla_lazy_attn_fwd replaces _lazy_attention_forward_return_lse
 * (lazy_attention_triton.py:543-583: kernels :9-88 and :90-174).
 * bias: float [H, bias_cols] with row stride bias_stride (elements); only columns < window
 * are read.  tau: float [H].  lse: float [B,H,L] out, the row log-sum-exp in base-2 units
 * (log2(e) times the natural one).  aux_o: float [B,H,L,2*D] or NULL (needed by the SIMT
 * family's backward, ignored by the tensor-core family): per row the fp32 output followed by
 * the sum of V rows over the ReLU support.  Rows at or beyond varlen are written as zeros (the
 * reference leaves them unwritten).                                                         */
int fla_lazy_attn_fwd(const fla_attn_geom* g, const fla_tensor4* q, const fla_tensor4* k,
                      const fla_tensor4* v, const fla_tensor4* o, const float* bias,
                      int64_t bias_stride, const float* tau, int32_t window, float* lse,
                      float* aux_o, void* stream);

size_t fla_lazy_attn_bwd_workspace(const fla_attn_geom* g);

/* fla_lazy_attn_bwd replaces _lazy_attention_backward (lazy_attention_triton.py:585-667) and,
 * with dbias == dtau == NULL, _lazy_attention_backward_fast (:670-745).
 * dbias: float [H, window] (row stride dbias_stride), dtau: float [H]; both are overwritten
 * (not accumulated), summed over the batch.  The sums are formed in 64-bit fixed point (32
 * fractional bits) inside the workspace and converted at the end, so they do not depend on the
 * order in which thread blocks arrive: repeated calls give bit-identical dbias and dtau, like
 * the reference's per-block buffers reduced in a fixed order (lazy_attention_triton.py:645-649). */
int fla_lazy_attn_bwd(const fla_attn_geom* g, const fla_tensor4* q, const fla_tensor4* k,
                      const fla_tensor4* v, const fla_tensor4* o, const fla_tensor4* dout,
                      const float* bias, int64_t bias_stride, const float* tau, int32_t window,
                      const float* lse, const float* aux_o, const fla_tensor4* dq,
                      const fla_tensor4* dk, const fla_tensor4* dv, float* dbias,
                      int64_t dbias_stride, float* dtau, void* workspace,
                      size_t workspace_bytes, void* stream);

/* ---- rotary position embedding of q and k -----------------------------------------------------
 * The step before the attention operators in the reference's layers (RotaryEmbedding of q and k,
 * examples/lazy_attention_layer.py:131, examples/sw_attention_lazy.py:150), as one launch over both
 * tensors.  Rotate-half convention over the head dimension: with x1 = x[..., :D/2], x2 = x[..., D/2:]
 * and angle(l, j) = (l + offset) / base^(j / (D/2)) in fp32,
 *   y1 = x1 cos - x2 sin,  y2 = x2 cos + x1 sin.
 * q_*: [B,Hq,L,D] views, k_*: [B,Hk,L,D] views or both NULL; inner stride 1, D even (16-byte accesses
 * when D is a multiple of 16 and bases and outer strides are 16-byte aligned, scalar ones otherwise);
 * out may alias in (in place).  inverse != 0 rotates back, which is also the gradient of the
 * rotation (it is orthogonal): dx = R^T dy.                                                   */
int fla_rope_qk(const fla_tensor4* q_in, const fla_tensor4* q_out, int32_t Hq, const fla_tensor4* k_in,
                const fla_tensor4* k_out, int32_t Hk, int32_t B, int32_t L, int32_t D, int32_t dtype,
                float base, int32_t offset, int32_t inverse, void* stream);

/* ---- self test of the tensor-core building blocks -----------------------------------------
 * No counterpart in the reference.  Computes C[128,128] (float) from bf16 A[128,128] and
 * B through one tcgen05 tile product, exercising one operand layout per `variant`:
 *   0: C = A . B^T, A and B K-major in shared memory (TMA, 128-byte swizzle)
 *   1: C = A . B,   B stored [K][N] (MN-major in shared memory)
 *   2: C = A . B^T, A read from tensor memory
 *   3: no product at all: the kernel waits, with a spin limit of a few thousand polls, on a
 *      barrier nothing arrives on, and leaves the way every kernel of this library leaves after
 *      an expired wait (status words set, tensor memory freed, normal return; C is zeroed).
 *      fla_check_status(status, stream) then reports FLA_ERR_DEVICE.  It exists so that this
 *      exit can be exercised without provoking a fault.
 * status: device int32[4] diagnostics, cleared by the call; status[0] != 0 if a bounded wait
 * ran out.                                                                                */
int fla_selftest_umma(const void* a, const void* b, float* c, int variant, int32_t* status,
                      void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLA_H_ */
