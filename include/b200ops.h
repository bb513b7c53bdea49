/*
 * b200ops.h -- C ABI of the sm_100a kernel library (libb200ops.so).
 *
 * This library takes the place that the closed vendor kernel library
 * (`topsaten::topsaten<Op>(out, in..., scalars..., stream)`) has in the
 * reference backend: the host code of the PrivateUse1 backend marshals every
 * at::Tensor into a non-owning {dims, strides, dtype, data} view and calls one
 * entry point per operator with the stream as the last argument
 * (reference: torch_gcu/csrc/aten/aot_ops/topsaten_bridge_define.h:323-427,
 * view construction torch_gcu/csrc/gcu/gcu_utils.cpp:79-108).
 *
 * Conventions
 *  - every entry point is `extern "C"`, re-entrant, and takes plain pointers
 *    and sizes only; no C++ or torch type crosses this boundary;
 *  - tensors are borrowed for the duration of the call; kernels are enqueued on
 *    `stream` (a cudaStream_t passed as void*) and the call returns without
 *    synchronising;
 *  - outputs are allocated by the caller (the host code runs ATen's meta
 *    functions, exactly as the reference's shape-inference layer does);
 *  - nothing in here allocates device memory: kernels that need scratch take a
 *    caller-supplied workspace whose size the matching *_workspace_size
 *    function reports;
 *  - every function returns a b200Status; b200_last_error() gives the
 *    thread-local message of the last non-OK status. The host maps non-OK to
 *    an exception (reference: CHECK_TOPSATEN_CALL, gcu_utils.cpp:64-77).
 *    Kernels never trap.
 *  - strides are in ELEMENTS, sizes/strides are int64, ndim <= 8; a rank-0
 *    tensor is passed with ndim == 0 (numel 1).
 */
#ifndef B200OPS_H_
#define B200OPS_H_

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library is built with hidden visibility */
#endif

#define B200_MAX_DIMS 8

typedef enum b200Status {
  B200_OK = 0,
  B200_BAD_PARAM = 1,           /* null pointer, shape/stride/dtype mismatch   */
  B200_NOT_SUPPORTED = 2,       /* valid request this library has no kernel for */
  B200_LAUNCH_FAILED = 3,       /* CUDA reported an error at enqueue            */
  B200_WORKSPACE_TOO_SMALL = 4,
  B200_TIMEOUT = 5
} b200Status;

typedef enum b200DType {
  B200_F32 = 0,
  B200_BF16 = 1,
  B200_F16 = 2,
  B200_F64 = 3,
  B200_I64 = 4,
  B200_I32 = 5,
  B200_I16 = 6,
  B200_I8 = 7,
  B200_U8 = 8,
  B200_BOOL = 9
} b200DType;

/* Non-owning strided view of device memory. */
typedef struct b200Tensor {
  void* data;
  int32_t dtype; /* b200DType */
  int32_t ndim;
  int64_t sizes[B200_MAX_DIMS];
  int64_t strides[B200_MAX_DIMS];
} b200Tensor;

typedef void* b200Stream; /* cudaStream_t */

/* ---- library / device queries ------------------------------------------- */
const char* b200_last_error(void);
const char* b200_version(void);
int b200_device_count(void);            /* 0 when no usable GPU / driver     */
int b200_sm_count(int device);          /* multiprocessors of `device`, or -1 */
size_t b200_dtype_size(int32_t dtype);  /* bytes per element, 0 if unknown    */
/* The persistent GEMM kernels fill every SM with one CTA whose shared memory
 * leaves no room for another kernel's CTA, so a collective launched beside them
 * on another stream would wait for the GEMM to end. Reserving n SMs makes those
 * kernels launch on (SM count - n) SMs; process-wide, default 0. No reference
 * counterpart (the vendor library schedules its own kernels).                  */
void b200_set_reserved_sms(int n);
/* Kernel launches this library has issued in this process so far (a counter for
 * benchmarks and tests: the difference around a region is the number of this
 * library's kernels launched inside it).                                        */
unsigned long long b200_launch_count(void);
int b200_get_reserved_sms(void);
/* Index kernels never trap on an out-of-range index: they substitute index 0
 * (or drop the element) and set bit 0 of a device-side error word. This call
 * synchronises the device, returns the word and clears it; the host uses it in
 * its per-op sync/debug mode (reference: op_sync_mode,
 * torch_gcu/csrc/gcu/gcu_stream.cpp:382-386).                                */
b200Status b200_device_error_fetch(uint32_t* flags);

/* ---- elementwise (reference: generated aotops::add_out / mul_out / silu_out
 *      -> topsatenAdd / topsatenMul / topsatenSilu; scalar-operand variants
 *      codegen/gen_backend_stubs.py:1061-1078) -------------------------------
 * Operands are broadcast against `out` by the caller (stride 0 on expanded
 * dims) and must already have out's dtype (type promotion is the host's job,
 * as TensorIterator does it in ATen's meta).                                 */
b200Status b200_add(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b,
                    double alpha, b200Stream stream); /* out = a + alpha*b     */
b200Status b200_mul(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b,
                    b200Stream stream);
b200Status b200_add_scalar(const b200Tensor* out, const b200Tensor* a, double b,
                           double alpha, b200Stream stream); /* a + alpha*b    */
b200Status b200_mul_scalar(const b200Tensor* out, const b200Tensor* a, double b,
                           b200Stream stream);
b200Status b200_silu(const b200Tensor* out, const b200Tensor* a, b200Stream stream);
/* Unary / binary helpers the unfused decoder layer reaches through the same
 * generated path (yaml rows neg.out, rsqrt.out, pow.Tensor_Scalar_out, ...). */
typedef enum b200UnaryOp {
  B200_UNARY_NEG = 0, B200_UNARY_RSQRT = 1, B200_UNARY_SQRT = 2, B200_UNARY_EXP = 3,
  B200_UNARY_SIGMOID = 4, B200_UNARY_TANH = 5, B200_UNARY_RELU = 6, B200_UNARY_ABS = 7,
  B200_UNARY_RECIPROCAL = 8, B200_UNARY_COS = 9, B200_UNARY_SIN = 10, B200_UNARY_LOG = 11,
  B200_UNARY_GELU = 12 /* erf form, as CPU ATen's default */
} b200UnaryOp;
b200Status b200_unary(const b200Tensor* out, const b200Tensor* a, int32_t op,
                      b200Stream stream);
b200Status b200_pow_scalar(const b200Tensor* out, const b200Tensor* a, double exponent,
                           b200Stream stream);
b200Status b200_sub(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b,
                    double alpha, b200Stream stream); /* out = a - alpha*b */
b200Status b200_div(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b,
                    b200Stream stream);
b200Status b200_fill(const b200Tensor* out, double value, b200Stream stream);
/* The same for an int64 tensor and an integer value that a double cannot carry (|value| > 2^53):
 * ATen keeps integer scalars exact.                                                   */
b200Status b200_fill_i64(const b200Tensor* out, int64_t value, b200Stream stream);

/* ---- copy / cast (reference: aotops::_copy_from -> copy_device_to_device ->
 *      topsatenCopy, torch_gcu/csrc/aten/aot_ops/gcu_copy.cpp:34-198,402-442)
 * dst[i] = (dst dtype) src[i] for same-shaped (caller-expanded) views; any
 * strides, any pair of dtypes. fp32->bf16 is round-to-nearest-even (NaN stays
 * NaN, payload unspecified).                               */
b200Status b200_copy(const b200Tensor* dst, const b200Tensor* src, b200Stream stream);

/* ---- reductions ---------------------------------------------------------- */
/* reference: generated aotops::sum_out -> topsatenSum. `dims` lists the reduced
 * dimensions of `in` (non-negative, unique); out has the reduced shape with or
 * without kept 1-dims (its numel decides nothing: only its data/dtype are used).
 * Accumulation is fp32 for f32/bf16/f16 inputs, fp64 for f64, int64 for ints. */
size_t b200_sum_workspace_size(const b200Tensor* in, const int64_t* dims, int32_t ndims);
b200Status b200_sum(const b200Tensor* out, const b200Tensor* in, const int64_t* dims,
                    int32_t ndims, int32_t mean /* 1: divide by count */,
                    void* workspace, size_t workspace_bytes, b200Stream stream);
/* reference: generated aotops::_softmax_out -> topsatenSoftmaxForward
 * (codegen/gcu_native_functions.yaml:182-183). out dtype may be f32 for a
 * bf16/f16 input (half_to_float).                                            */
b200Status b200_softmax(const b200Tensor* out, const b200Tensor* in, int64_t dim,
                        b200Stream stream);
/* reference: aotops::native_layer_norm -> topsatenNativeLayerNorm
 * (torch_gcu/csrc/aten/aot_ops/gcu_layer_norm.cpp:17-86). `in` is viewed as
 * (M, N) contiguous, N = product of normalized_shape; weight/bias may be NULL;
 * mean/rstd are (M) tensors in the accumulate type (f32) or in's dtype.       */
b200Status b200_native_layer_norm(const b200Tensor* out, const b200Tensor* mean,
                                  const b200Tensor* rstd, const b200Tensor* in,
                                  int64_t M, int64_t N, const b200Tensor* weight,
                                  const b200Tensor* bias, double eps, b200Stream stream);

/* ---- index ops ----------------------------------------------------------- */
/* reference: generated aotops::index_select -> topsatenIndexSelect (this is
 * also where aten::embedding lands). index: 1-D int32/int64.                 */
b200Status b200_index_select(const b200Tensor* out, const b200Tensor* self, int64_t dim,
                             const b200Tensor* index, b200Stream stream);
/* reference: generated aotops::gather_out -> topsatenGather.                  */
b200Status b200_gather(const b200Tensor* out, const b200Tensor* self, int64_t dim,
                       const b200Tensor* index, b200Stream stream);
/* reference: generated aotops::scatter_add_out -> topsatenScatterAdd.
 * out = self; out[index[i][j]][j] += src[i][j] (for dim 0; any dim accepted).
 * Every destination element receives its addends in ascending source order
 * along `dim`, starting from self's value -- the order CPU ATen uses -- so the
 * result is bit-identical to the CPU's and run-to-run reproducible. out may
 * alias self.                                                                */
size_t b200_scatter_add_workspace_size(const b200Tensor* self, int64_t dim,
                                       const b200Tensor* index, const b200Tensor* src);
b200Status b200_scatter_add(const b200Tensor* out, const b200Tensor* self, int64_t dim,
                            const b200Tensor* index, const b200Tensor* src,
                            void* workspace, size_t workspace_bytes, b200Stream stream);
/* No counterpart in the reference. The same deterministic scatter_add for
 * callers that must not allocate device memory while they run: code inside a
 * region where cudaMalloc is forbidden or would serialise the device (a latency
 * critical serving loop, a caller that owns no allocator, a plugin handed only
 * input and output buffers). It takes no workspace: its scratch is a fixed 8 MiB
 * array inside the library (held by every GPU that loads the library, until
 * exit), enough for about 470 000 source rows in the row-index form; a larger
 * problem is refused with B200_NOT_SUPPORTED and a message that says how much
 * was needed. It calls no allocation routine of any kind.
 * - The first call on each device looks up the array's device address; make
 *   that first call before starting any stream capture on that device.
 * - Every call uses the same array, so two calls whose kernels can overlap on
 *   the GPU (different streams, different host threads) race: serialise them.
 *   The array keeps the previous call's contents; nothing in it needs clearing
 *   between calls, every call rewrites all it reads.                          */
b200Status b200_scatter_add_static(const b200Tensor* out, const b200Tensor* self, int64_t dim,
                                   const b200Tensor* index, const b200Tensor* src,
                                   b200Stream stream);
/* reference: aotops::_index_put_impl_ -> topsatenIndexPutImpl
 * (torch_gcu/csrc/aten/aot_ops/gcu_tensor_advanced_indexing.cpp:60-90).
 * self[index[i], ...] (+)= values[i, ...] for ONE index tensor over the
 * leading dimension of a contiguous self (the host reduces the general case to
 * this by linearising the indexed dims). accumulate != 0 adds in ascending i
 * order (bit-identical to CPU ATen under deterministic algorithms);
 * accumulate == 0 writes and, on duplicates, the highest i wins.             */
size_t b200_index_put_workspace_size(const b200Tensor* self, const b200Tensor* index,
                                     const b200Tensor* values);
b200Status b200_index_put(const b200Tensor* self, const b200Tensor* index,
                          const b200Tensor* values, int32_t accumulate,
                          void* workspace, size_t workspace_bytes, b200Stream stream);
/* reference: efficient::device_int32_indices_index -> topsatenIndex
 * (torch_gcu/csrc/efficient_ops/ops.cpp:335-342) and aotops index
 * (gcu_tensor_advanced_indexing.cpp:40-58). Arguments are ATen's AdvancedIndex
 * (ops.cpp:48-90): `src` is self restrided to out's shape with stride 0 on the
 * indexed dims, `indices[k]` are int32 or int64 tensors broadcast to out's
 * shape, and indexed_sizes/strides (elements) describe the replaced dims.
 * Negative indices wrap once, as in ATen.                                    */
b200Status b200_index(const b200Tensor* out, const b200Tensor* src,
                      const b200Tensor* const* indices, int32_t n_indices,
                      const int64_t* indexed_sizes, const int64_t* indexed_strides,
                      b200Stream stream);

/* ---- contractions (reference: generated aotops::mm_out / addmm_out / bmm_out
 *      -> topsatenMm / topsatenAddmm / topsatenBmm / topsatenBaddbmm) ----------
 * out = beta*self + alpha*(a @ b). bf16 / f16 operands run on the tcgen05 tensor
 * cores with fp32 accumulation and one rounding of the result; each operand may
 * be row- or column-major (e.g. `weight.t()`) as long as its leading dimension
 * is a multiple of 8 elements and its base 16-byte aligned, and out's last
 * dimension is contiguous. fp32 / fp64 and every other layout take an exact-order
 * SIMT kernel. `self` must be expanded to out's shape by the caller.          */
b200Status b200_mm(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b,
                   b200Stream stream);
b200Status b200_addmm(const b200Tensor* out, const b200Tensor* self, const b200Tensor* a,
                      const b200Tensor* b, double beta, double alpha, b200Stream stream);
b200Status b200_bmm(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b,
                    b200Stream stream);
b200Status b200_baddbmm(const b200Tensor* out, const b200Tensor* self, const b200Tensor* a,
                        const b200Tensor* b, double beta, double alpha, b200Stream stream);

/* reference: aotops::_scaled_dot_product_flash_attention ->
 * topsatenScaledDotProductFlashAttention (torch_gcu/csrc/aten/aot_ops/
 * gcu_attention.cpp:21-80; backend choice RegisterSPDA.cpp:223-275).
 * q (B,Hq,Sq,D), k/v (B,Hkv,Sk,D), out like q (any strides with D contiguous, so
 * the (B,S,H,D)-allocated, transposed output of the reference's shape inference
 * is written in place), lse f32 (B,Hq,Sq) or NULL. bf16/f16, D 64 or 128, Hq a
 * multiple of Hkv. is_causal needs Sq == Sk; dropout is not supported.         */
b200Status b200_sdpa_flash_fwd(const b200Tensor* out, const b200Tensor* lse, const b200Tensor* q,
                               const b200Tensor* k, const b200Tensor* v, int32_t is_causal,
                               double scale, b200Stream stream);

/* ---- fused inference ops (no counterpart kernel in the reference, which runs
 *      them as chains of the ops above; they sit beside the reference's one
 *      efficient op, torch_gcu/csrc/efficient_ops/ops.cpp:335-342) ---------- */
/* h = x + residual (rounded to the I/O dtype, written to residual_out);
 * y = h * rsqrt(mean(h^2) + eps) * weight, fp32 internally. x/residual: (M,N)
 * contiguous bf16/f16/f32. residual may be NULL (plain RMSNorm). Outputs may
 * alias the inputs.                                                          */
b200Status b200_rms_norm_residual(const b200Tensor* y, const b200Tensor* residual_out,
                                  const b200Tensor* x, const b200Tensor* residual,
                                  const b200Tensor* weight, double eps, b200Stream stream);
/* Rotate-half rotary embedding (the Llama / HF convention):
 * out[..., i]       = x[..., i]*cos[p,i] - x[..., i+D/2]*sin[p,i]
 * out[..., i+D/2]   = x[..., i+D/2]*cos[p,i] + x[..., i]*sin[p,i],  i < D/2,
 * x: (B,S,H,D) with D contiguous; cos/sin: f32 (P, D/2) tables; positions:
 * int64 (B,S) or NULL for p = s. fp32 math, one rounding. In place allowed.   */
b200Status b200_rope(const b200Tensor* out, const b200Tensor* x, const b200Tensor* cos_table,
                     const b200Tensor* sin_table, const b200Tensor* positions,
                     b200Stream stream);
/* Rotary embedding of a decode step fused with the write into the KV cache: qkv is a fused projection
 * output (B, S, q_heads + 2 k_heads, D), D contiguous. Query heads are rotated in place; key heads are
 * rotated (the arithmetic of b200_rope, bit for bit) and written to k_cache[b, head, p, :]; value heads
 * are copied to v_cache[b, head, p, :], with p = positions[b, s] (int64 (B,S)) both the row of the
 * cos / sin tables (f32 (P, D/2)) and the slot of the caches ((B, k_heads, T, D) views, D contiguous).
 * The key and value parts of qkv are left as they were. A position outside [0, min(P, T)) writes
 * nothing and sets bit 0 of the device error word. Replaces b200_rope followed by two strided copies.
 * No reference counterpart.                                                                          */
b200Status b200_rope_kv_append(const b200Tensor* qkv, const b200Tensor* cos_table,
                               const b200Tensor* sin_table, const b200Tensor* positions,
                               int64_t q_heads, int64_t k_heads, const b200Tensor* k_cache,
                               const b200Tensor* v_cache, b200Stream stream);
/* out = silu(gate) * up, fp32 math, one rounding. 2-D views with contiguous
 * last dim (gate and up may be the two halves of one projection output).      */
b200Status b200_swiglu(const b200Tensor* out, const b200Tensor* gate, const b200Tensor* up,
                       b200Stream stream);
/* Gate/up projection with the SwiGLU fused into the GEMM epilogue:
 *   out (M,F) = silu(a @ w[0:F].T) * (a @ w[F:2F].T),
 * a (M,K) and w (2F,K) bf16 / f16 with K contiguous (the nn.Linear weight of a
 * fused gate/up projection, gate rows first). The activation is evaluated on the
 * fp32 accumulators and rounded once; the (M,2F) intermediate is never written.
 * No reference counterpart: the reference runs mm followed by pointwise ops.     */
b200Status b200_mm_swiglu(const b200Tensor* out, const b200Tensor* a, const b200Tensor* w_gate_up,
                          b200Stream stream);
/* 1 when b200_mm_swiglu has a kernel made for few rows (M <= 128) against this weight: one wave of
 * equal tiles, one per SM, for a wide weight, or K split over clusters with the activation applied
 * by the CTA that sums a band, for a narrower one; both stream the weight once. 0 when it would
 * fall back to the 256-row pair tiles, which for so few rows are slower than b200_mm followed by
 * b200_swiglu. Lets a caller pick without repeating the kernels' tile rules. No reference
 * counterpart.                                                                                   */
int b200_mm_swiglu_few_rows(int64_t M, int64_t F, int64_t K);
/* Fused qkv projection with the rotary embedding in the GEMM epilogue:
 *   out (M,N) = a @ w^T, then rotate-half RoPE (the convention of b200_rope) on the first
 *   rope_cols columns, taken as heads of 128; row m has position m % seq_len.
 * a (M,K), w (N,K) bf16 / f16 with K contiguous; cos / sin f32 (positions, 64). The rotation
 * acts on the fp32 accumulators, one rounding. No reference counterpart.                 */
b200Status b200_mm_rope(const b200Tensor* out, const b200Tensor* a, const b200Tensor* w,
                        const b200Tensor* cos_table, const b200Tensor* sin_table, int64_t seq_len,
                        int64_t rope_cols, b200Stream stream);

/* ---- comparison, selection, clamping, extremes, generators ------------------
 * The operators model code needs around the hot path (masks, sampling, position
 * ids); they take the place of the vendor calls behind the reference's generated
 * aotops::eq_out … ge_out, where, masked_fill_, maximum_out, clamp_out, argmax_out,
 * max.dim, arange_out, triu_out / tril_out (rows of codegen/gcu_native_functions.yaml).
 * Semantics are CPU ATen's: comparisons with NaN are false (NE true); maximum,
 * minimum and clamp propagate NaN; extremes return the first occurrence, and the
 * first NaN if there is one.                                                      */
enum b200CompareOp {
  B200_CMP_EQ = 0, B200_CMP_NE, B200_CMP_LT, B200_CMP_LE, B200_CMP_GT, B200_CMP_GE,
  B200_CMP_AND, B200_CMP_OR, B200_CMP_XOR   /* logical, operands tested against zero */
};
/* out (bool) = a <op> b; a and b of one dtype (any arithmetic dtype or bool),
 * expanded to out's shape.                                                        */
b200Status b200_compare(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b, int32_t op,
                        b200Stream stream);
/* out (bool) = a <op> scalar, the scalar rounded to a's dtype first.               */
b200Status b200_compare_scalar(const b200Tensor* out, const b200Tensor* a, double b, int32_t op,
                               b200Stream stream);
/* out = cond ? a : b (cond bool; a, b, out one dtype; all expanded to out's shape). */
b200Status b200_where(const b200Tensor* out, const b200Tensor* cond, const b200Tensor* a,
                      const b200Tensor* b, b200Stream stream);
/* out = mask ? value : self. In place allowed.                                     */
b200Status b200_masked_fill(const b200Tensor* out, const b200Tensor* self, const b200Tensor* mask,
                            double value, b200Stream stream);
/* out = max(a, b) (is_max) or min(a, b), elementwise.                              */
b200Status b200_minmax(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b, int32_t is_max,
                       b200Stream stream);
/* out = clamp(a, min, max) with either bound optional (has_min / has_max).         */
b200Status b200_clamp(const b200Tensor* out, const b200Tensor* a, int32_t has_min, double min_value,
                      int32_t has_max, double max_value, b200Stream stream);
/* Maximum (is_max) or minimum of a contiguous tensor along `dim`: values (input's
 * dtype) and / or indices (int64), each contiguous with the reduced dim removed;
 * either may be NULL.                                                              */
b200Status b200_extreme_dim(const b200Tensor* values, const b200Tensor* indices, const b200Tensor* in,
                            int64_t dim, int32_t is_max, b200Stream stream);
/* out[i] = start + i * step (1-D contiguous; integer outputs computed in int64).   */
b200Status b200_arange(const b200Tensor* out, double start, double step, b200Stream stream);
/* Upper (upper != 0) or lower triangle of the last two dims of a contiguous tensor,
 * zeros elsewhere; `diagonal` as in torch.triu / torch.tril. In place allowed.      */
b200Status b200_tri(const b200Tensor* out, const b200Tensor* in, int64_t diagonal, int32_t upper,
                    b200Stream stream);

/* ---- sort, top-k, cumulative sum (what a sampling step needs around the logits) ----
 * reference: generated aotops::sort_out / argsort / topk_out / cumsum_out -> the vendor's
 * sort, topk and cumsum calls (codegen/gcu_native_functions.yaml rows sort.values_stable,
 * argsort.stable, topk.values, cumsum.out).
 * b200_sort_rows: stable sort of every row of a contiguous (rows, n) tensor, ascending or
 * descending; NaN orders above every number and -0 equals +0, as in CPU ATen; equal elements
 * keep their input order. values (in's dtype) and / or indices (int64), each contiguous
 * (rows, k) with k <= n, take the first k sorted entries of every row (k = n: sort / argsort;
 * k < n with descending: topk largest, ties by lowest index). Either output may be NULL.    */
size_t b200_sort_rows_workspace_size(const b200Tensor* in);
b200Status b200_sort_rows(const b200Tensor* values, const b200Tensor* indices, const b200Tensor* in,
                          int32_t descending, void* workspace, size_t workspace_bytes, b200Stream stream);
/* out[..., i, ...] = sum of in[..., 0..i, ...] along `dim`; contiguous operands of one dtype.
 * Accumulates as CPU ATen does: fp32 in fp64, bf16 / f16 in fp32, integers in int64. Along a
 * non-last dimension the additions run in index order (bit-identical to the CPU); along the
 * last dimension the row is scanned in parallel (fp results within an ulp of the CPU's,
 * integers identical).                                                                    */
b200Status b200_cumsum(const b200Tensor* out, const b200Tensor* in, int64_t dim, b200Stream stream);

/* ---- backward of the layer's pointwise and row operators ---------------------
 * (reference yaml rows silu_backward.grad_input, _softmax_backward_data.out,
 * native_layer_norm_backward; fp32 math, one rounding per output, reductions in a
 * fixed order.)                                                                    */
/* grad_in = grad_out * s * (1 + x * (1 - s)), s = sigmoid(x).                      */
b200Status b200_silu_backward(const b200Tensor* grad_in, const b200Tensor* grad_out, const b200Tensor* x,
                              b200Stream stream);
/* grad_in = output * (grad_out - sum_dim(grad_out * output)); contiguous operands.  */
b200Status b200_softmax_backward(const b200Tensor* grad_in, const b200Tensor* grad_out,
                                 const b200Tensor* output, int64_t dim, b200Stream stream);
/* Layer-norm backward over an (M, N) view: dx, dweight, dbias (each optional) from
 * grad_out, x, the saved f32 mean / rstd (M each) and the optional weight. dweight
 * and dbias need a workspace of b200_layer_norm_backward_workspace_size bytes.      */
size_t b200_layer_norm_backward_workspace_size(int64_t M, int64_t N);
b200Status b200_layer_norm_backward(const b200Tensor* dx, const b200Tensor* dweight, const b200Tensor* dbias,
                                    const b200Tensor* grad_out, const b200Tensor* x, const b200Tensor* mean,
                                    const b200Tensor* rstd, const b200Tensor* weight, int64_t M, int64_t N,
                                    void* workspace, size_t workspace_bytes, b200Stream stream);

/* Log-softmax along `dim` and its backward (grad_in = grad_out - exp(output) * sum(grad_out));
 * negative log-likelihood over (N, C) log-probabilities with int64 targets, optional
 * class weights, ignore_index, reduction 0 none / 1 mean / 2 sum, and its backward
 * (reference yaml rows _log_softmax.out, _log_softmax_backward_data.out,
 * nll_loss_forward.output, nll_loss_backward.grad_input). Contiguous operands.        */
b200Status b200_log_softmax(const b200Tensor* out, const b200Tensor* in, int64_t dim, b200Stream stream);
b200Status b200_log_softmax_backward(const b200Tensor* grad_in, const b200Tensor* grad_out,
                                     const b200Tensor* output, int64_t dim, b200Stream stream);
b200Status b200_nll_loss(const b200Tensor* out, const b200Tensor* total_weight, const b200Tensor* logp,
                         const b200Tensor* target, const b200Tensor* weight, int32_t reduction,
                         int64_t ignore_index, b200Stream stream);
b200Status b200_nll_loss_backward(const b200Tensor* grad_in, const b200Tensor* grad_out,
                                  const b200Tensor* target, const b200Tensor* weight,
                                  const b200Tensor* total_weight, int32_t reduction, int64_t ignore_index,
                                  b200Stream stream);
/* Flash-attention backward (reference: aot_ops/gcu_attention.cpp:135-203
 * topsatenScaledDotProductFlashAttentionBackward). dq (B,Hq,Sq,D), dk / dv
 * (B,Hkv,Sk,D) from dout, q, k, v, the forward's out and logsumexp; D = 128,
 * bf16 / f16, last dim contiguous, other strides free, causal needs Sq == Sk.
 * The probabilities are recomputed from q, k and lse; no atomics are used, so
 * the gradients are reproducible. Needs b200_sdpa_flash_bwd_workspace_size(q)
 * bytes of workspace (the per-row sum of dout * out).                            */
size_t b200_sdpa_flash_bwd_workspace_size(const b200Tensor* q);
b200Status b200_sdpa_flash_bwd(const b200Tensor* dq, const b200Tensor* dk, const b200Tensor* dv,
                               const b200Tensor* dout, const b200Tensor* q, const b200Tensor* k,
                               const b200Tensor* v, const b200Tensor* out, const b200Tensor* lse,
                               int32_t is_causal, double scale, void* workspace, size_t workspace_bytes,
                               b200Stream stream);

/* ---- tensor-parallel exchange over peer memory ---------------------------------------
 * What stands where the reference's row-parallel projections call the collective library
 * (reference: torch_gcu/csrc/distributed/ProcessGroupECCL.cpp:2869-2926 allreduce, :3326-3432
 * reduce_scatter, :3077-3166 allgather): this library's own kernels, over plain peer loads and
 * stores. Every rank maps the other ranks' buffers once (IPC handles; the host's job) and
 * passes a table of base addresses as seen from THIS process, its own buffer at [rank].       */
#define B200_TP_MAX_RANKS 8
typedef struct b200TpPeers {
  int32_t world; /* ranks, 1..B200_TP_MAX_RANKS */
  int32_t rank;  /* this rank                  */
  void* base[B200_TP_MAX_RANKS];
} b200TpPeers;
/* Bytes of one rank's control block (flags and counters of b200_tp_sync); the host allocates one
 * per rank in peer-visible memory, zeroes it once before first use, and passes the table.       */
size_t b200_tp_control_bytes(void);
/* Counting signal / wait between the ranks on `channel` (0..15). do_signal: every peer's copy of
 * this rank's flag takes this rank's next count, after a system-scope fence, so what this GPU
 * wrote earlier on the stream is visible to a peer that has seen the flag. do_wait: returns once
 * every peer has signalled this channel as often as this rank has waited on it. Both in one
 * call is a barrier. Counts live in the control block, so a captured graph replays correctly.
 * The wait is bounded: after timeout_ns (> 0) it sets bit 1 (TIMEOUT) of the device error word
 * (b200_device_error_fetch) and returns; the control blocks must then be zeroed again on every
 * rank before further use. A channel must not be used from two streams at once.                */
b200Status b200_tp_sync(const b200TpPeers* control, int32_t channel, int32_t do_signal, int32_t do_wait,
                        uint64_t timeout_ns, b200Stream stream);
/* Reduce-scatter + residual add + RMSNorm + all-gather of one row-parallel projection in one
 * kernel. partial->base[r]: rank r's partial product, (total_rows, N) bf16 / f16 row-major (NULL
 * table: nothing to reduce). This rank owns rows [row0, row0 + rows), rows = residual's row
 * count: for each it sums the row of every rank's partial in fp32 in rank order, adds `residual`
 * (rows, N; may be NULL), rounds once -> residual_out (rows, N; may alias residual; may be NULL),
 * normalises with `weight` (N) and eps when normalise != 0, and stores the row at
 * gathered->base[r] + row offset for every rank r (gather_all != 0) or only for this rank.
 * The caller orders it between b200_tp_sync calls: partials complete on every rank before, the
 * gathered rows complete on every rank after.                                                  */
b200Status b200_tp_reduce_norm(const b200TpPeers* partial, const b200TpPeers* gathered,
                               const b200Tensor* residual, const b200Tensor* residual_out,
                               const b200Tensor* weight, int64_t row0, int64_t total_rows, double eps,
                               int32_t normalise, int32_t gather_all, b200Stream stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* B200OPS_H_ */
