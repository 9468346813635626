/*
 * b200ops.h -- C ABI of libb200ops.so: hand-written sm_100a CUDA kernels for the
 * sixteen ATen operators that a BackendBench directory backend overrides, plus the
 * two device-side helpers of the evaluation path (allclose/error scan, L2 flush).
 *
 * The reference project (meta-pytorch/BackendBench) is pure Python and has no FFI
 * of its own: the arithmetic it checks against is `torch.ops.aten.<op>` reached at
 * BackendBench/eval.py:100 (reference result) and BackendBench/eval.py:102 (the
 * backend's `impl(*args, **kwargs)`). Every entry point below is what the
 * `<folder>_kernel_impl` function loaded by BackendBench/backends/directory.py:74-100
 * binds for one aten overload; the citation on each declaration names the aten
 * overload and the reference call site it replaces.
 *
 * Conventions (all entry points):
 *   - return 0 on success, a negative B200_E* code otherwise; never throw;
 *   - all `void*` tensor arguments are DEVICE pointers owned by the caller, valid
 *     in the CUDA context current on the calling thread;
 *   - nothing is allocated and nothing is synchronised: the work is enqueued on
 *     `stream` (a cudaStream_t passed as void*; NULL = the legacy default stream);
 *   - sizes and strides are in ELEMENTS, int64, host arrays read before return;
 *   - `dtype` arguments take the b200_dtype codes below;
 *   - index-taking kernels record an out-of-range index in `*status` (a 4-byte
 *     device word, may be NULL) instead of faulting: the bad row/element is
 *     written as zero / skipped and B200_DEV_INDEX_OOB is OR-ed into the word.
 */
#ifndef B200OPS_H
#define B200OPS_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ABI_VERSION 1
#define B200_MAX_DIMS 8

typedef enum {
  B200_F32 = 0,
  B200_BF16 = 1,
  B200_F16 = 2,
  B200_I32 = 3,
  B200_I64 = 4,
  B200_BOOL = 5,
  B200_U8 = 6,
  B200_I8 = 7,
  B200_I16 = 8,
  B200_F64 = 9
} b200_dtype;

/* host-side return codes */
#define B200_OK 0
#define B200_EINVAL (-1)      /* bad argument (null pointer, negative size, rank > B200_MAX_DIMS) */
#define B200_EDTYPE (-2)      /* dtype combination not implemented */
#define B200_ELAUNCH (-3)     /* kernel launch failed; see b200_last_cuda_error() */
#define B200_ESCRATCH (-4)    /* scratch buffer too small / beyond the static maximum */
#define B200_EALIGN (-5)      /* pointer or stride alignment unusable for this path */
#define B200_EDRIVER (-6)     /* a driver entry point (tensor-map encode) was unavailable */

/* bits OR-ed into a device status word */
#define B200_DEV_INDEX_OOB 1u /* an index was outside [0, size) */
#define B200_DEV_WAIT_TIMEOUT 2u /* a bounded mbarrier wait gave up */

int b200_abi_version(void);
const char* b200_strerror(int code);
/* cudaGetErrorString of the last failing launch seen by this library on this thread. */
const char* b200_last_cuda_error(void);
/* Kernels (and device-to-device copies) this library has enqueued since it was loaded;
 * the benchmark reports the difference across its timed region. */
long long b200_launch_count(void);

/* ----------------------------------------------------------------- elementwise
 * Operands are described TensorIterator-style: one broadcast `shape[ndim]` and one
 * stride array per operand (stride 0 = broadcast). `out` is contiguous in `shape`.
 * Contiguous same-dtype 16-byte-aligned operands take the vectorised path.      */

/* aten.relu.default(self)  -- reference call site BackendBench/eval.py:100-102;
 * pinned by test/test_monkey_patch.py:99-100 and test/test_directory_backend.py:35-45. */
int b200_relu(const void* x, void* out, int ndim, const int64_t* shape, const int64_t* sx,
              int dtype, void* stream);

/* aten.add.Tensor(self, other, *, alpha=1): out = a + alpha*b computed in fp32,
 * rounded once to dtype_out (eval.py:100-102; test/test_directory_backend.py:48-58). */
int b200_add(const void* a, const void* b, void* out, int ndim, const int64_t* shape,
             const int64_t* sa, const int64_t* sb, int dtype_a, int dtype_b, int dtype_out,
             double alpha, void* stream);

/* aten.mul.Tensor(self, other) (eval.py:100-102; test/test_directory_backend.py:61-71). */
int b200_mul(const void* a, const void* b, void* out, int ndim, const int64_t* shape,
             const int64_t* sa, const int64_t* sb, int dtype_a, int dtype_b, int dtype_out,
             void* stream);

/* add.Tensor / mul.Tensor when `other` is a wrapped number (`x + 2.0` reaches the CUDA
 * kernel as a 0-dim CPU tensor): out = x + value (value = alpha*other) or x * value. */
int b200_add_scalar(const void* x, void* out, int ndim, const int64_t* shape, const int64_t* sx,
                    int dtype_x, int dtype_out, double value, void* stream);
int b200_mul_scalar(const void* x, void* out, int ndim, const int64_t* shape, const int64_t* sx,
                    int dtype_x, int dtype_out, double value, void* stream);

/* aten.where.self(condition, self, other): cond is bool/u8 (eval.py:100-102). */
int b200_where(const void* cond, const void* x, const void* y, void* out, int ndim,
               const int64_t* shape, const int64_t* sc, const int64_t* sx, const int64_t* sy,
               int dtype_x, int dtype_y, int dtype_out, void* stream);

/* Strided -> contiguous copy with optional float dtype conversion; the host side uses
 * it to materialise transposed / expanded inputs for the row kernels (no aten call). */
int b200_copy_strided(const void* x, void* out, int ndim, const int64_t* shape,
                      const int64_t* sx, int dtype_in, int dtype_out, void* stream);

/* [batch, rows, cols] copy from arbitrary element strides into a destination with unit
 * column stride and the given row / batch pitches (elements); elem_size 2 or 4. The host
 * side uses it to give a misaligned 16-bit GEMM operand a TMA-compatible row pitch. */
int b200_copy_pitched(const void* x, void* out, int64_t batch, int64_t rows, int64_t cols,
                      int64_t sx_batch, int64_t sx_row, int64_t sx_col, int64_t out_batch_pitch,
                      int64_t out_row_pitch, int elem_size, void* stream);

/* Bit-exact copy between two strided layouts of one shape (element strides sx -> so): how
 * the host writes a result into a caller-provided non-contiguous tensor, i.e. the `.out`
 * and in-place overloads that BackendBench/scripts/op_map.py:7-1148 lists next to each
 * functional operator. elem_size 1, 2, 4 or 8. Source and destination must not overlap. */
int b200_copy_into(const void* x, void* out, int ndim, const int64_t* shape, const int64_t* sx,
                   const int64_t* so, int elem_size, void* stream);

/* ----------------------------------------------------------------- row kernels
 * The input is contiguous and viewed as [outer, dim, inner]; the op runs along `dim`. */

/* aten._softmax.default / aten._log_softmax.default (self, dim, half_to_float):
 * fp32 internal math; dtype_out == dtype_in, or F32 when half_to_float (eval.py:100-102). */
int b200_softmax(const void* x, void* out, int64_t outer, int64_t dim, int64_t inner,
                 int dtype_in, int dtype_out, int log_softmax, void* stream);

/* aten._softmax_backward_data.default / aten._log_softmax_backward_data.default
 * (grad_output, output, dim, input_dtype), the operators BackendBench/backends/flag_gems.py:196,233
 * lists next to the forward ones:
 *   softmax:      grad_input = (grad - sum(grad * output)) * output
 *   log_softmax:  grad_input = grad - exp(output) * sum(grad)
 * along `dim` of the contiguous [outer, dim, inner] view; grad and output share dtype_in,
 * grad_input has dtype_out (= input_dtype); fp32 internal math. */
int b200_softmax_backward(const void* grad, const void* output, void* grad_input, int64_t outer,
                          int64_t dim, int64_t inner, int dtype_in, int dtype_out,
                          int log_softmax, void* stream);

/* Scratch size (bytes, possibly 0) that b200_sum / b200_argmax need for this geometry:
 * when few output elements face a long reduction, the reduction is split across CTAs
 * and per-split partials (fp32 sum, or fp32 value + int64 index) are staged there. */
int64_t b200_reduce_scratch_bytes(int64_t outer, int64_t dim, int64_t inner);

/* aten.sum.dim_IntList(self, dim, keepdim, *, dtype): fp32 accumulation, one rounding.
 * `scratch` (device, >= b200_reduce_scratch_bytes) may be NULL when that size is 0. */
int b200_sum(const void* x, void* out, int64_t outer, int64_t dim, int64_t inner,
             int dtype_in, int dtype_out, void* scratch, int64_t scratch_bytes, void* stream);

/* Same result as b200_sum, for hosts that must not allocate. It has no counterpart in
 * the reference: it exists for callers that drive this library from C/C++ (or through
 * cgo / JNI) without a device allocator of their own -- a serving loop whose GPU memory
 * was handed over to another pool at start-up, or code on a latency path where
 * cudaMalloc / cudaFree would stall the whole device. Such a caller passes only the input
 * and the output; the partial sums of a split reduction go to a fixed array inside the
 * library image (B200_STATIC_SCRATCH_BYTES per GPU that loads the library, held until the
 * process exits). The call allocates nothing and calls no allocating routine.
 *   - Geometries whose partials would not fit (b200_reduce_scratch_bytes(...) >
 *     B200_STATIC_SCRATCH_BYTES) are refused with B200_ESCRATCH; nothing is launched.
 *   - The first call on each device looks up the array's device address; make that first
 *     call with the device current and before starting any stream capture.
 *   - All calls on a device share the one array. Its old contents never matter (every
 *     partial is rewritten before it is read), but two calls whose kernels may run at the
 *     same time -- different streams, different host threads -- race on it: keep such
 *     calls ordered on one stream. */
#define B200_STATIC_SCRATCH_BYTES (1 << 20)
int b200_sum_static(const void* x, void* out, int64_t outer, int64_t dim, int64_t inner,
                    int dtype_in, int dtype_out, void* stream);

/* aten.native_layer_norm.default(input, normalized_shape, weight, bias, eps)
 * -> (out, mean, rstd); rows = prod(leading dims), cols = prod(normalized_shape);
 * weight/bias may be NULL; dtype_stat is the dtype of mean/rstd (eval.py:100-102;
 * output convention as BackendBench/backends/flag_gems.py:19-31). */
int b200_layer_norm(const void* x, const void* weight, const void* bias, void* y, void* mean,
                    void* rstd, int64_t rows, int64_t cols, double eps, int dtype,
                    int dtype_wb, int dtype_stat, void* stream);

/* aten.native_layer_norm_backward.default(grad_out, input, normalized_shape, mean, rstd,
 * weight, bias, output_mask) -- the backward neighbour at BackendBench/backends/flag_gems.py:140.
 * With xhat = (x - mean) * rstd and gy = dy * weight per row:
 *   dx = rstd * (gy - mean_j(gy) - xhat * mean_j(gy * xhat)); dw = sum_rows dy * xhat; db = sum_rows dy.
 * dx / dw / db may each be NULL (output_mask); weight may be NULL. dw / db need
 * b200_layer_norm_backward_scratch_bytes(rows, cols) bytes of scratch (per-CTA partials). */
int64_t b200_layer_norm_backward_scratch_bytes(int64_t rows, int64_t cols);
int b200_layer_norm_backward(const void* dy, const void* x, const void* mean, const void* rstd,
                             const void* weight, void* dx, void* dw, void* db, int64_t rows,
                             int64_t cols, int dtype, int dtype_wb, int dtype_stat, void* scratch,
                             int64_t scratch_bytes, void* stream);

/* aten.argmax.default(self, dim, keepdim): int64 index of the first maximum along
 * `dim`, NaN counts as the maximum (eval.py:100-102). dim must be > 0. */
int b200_argmax(const void* x, int64_t* out, int64_t outer, int64_t dim, int64_t inner,
                int dtype, void* scratch, int64_t scratch_bytes, void* stream);

/* -------------------------------------------------------------------- indexing */

/* aten.embedding.default(weight, indices, ...) and aten.index_select.default(self, 0, index)
 * on a contiguous table: out[i, :] = table[idx[i], :]; rows are `row_bytes` long
 * (bit copy, any dtype). idx_dtype is B200_I32 or B200_I64 (eval.py:100-102). */
int b200_gather_rows(const void* table, const void* idx, void* out, int64_t table_rows,
                     int64_t row_bytes, int64_t n_idx, int idx_dtype, uint32_t* status,
                     void* stream);

/* aten.index_select.default(self, dim, index) for dim != 0: self contiguous viewed as
 * [outer, dim_size, inner]; out is [outer, n_idx, inner]; elem_size in bytes. */
int b200_index_select(const void* x, const void* idx, void* out, int64_t outer,
                      int64_t dim_size, int64_t inner, int64_t n_idx, int elem_size,
                      int idx_dtype, uint32_t* status, void* stream);

/* aten.gather.default(self, dim, index): out (contiguous, index's shape)
 * out[p] = self[p with p[dim] := index[p]]; bit copy of elem_size bytes (eval.py:100-102). */
int b200_gather(const void* self, const void* index, void* out, int ndim,
                const int64_t* index_shape, const int64_t* self_strides,
                const int64_t* index_strides, int64_t self_dim_size, int dim, int elem_size,
                uint32_t* status, void* stream);

/* aten.scatter_add.default(self, dim, index, src): out = self, then for every p in
 * index's shape out[p with p[dim] := index[p]] += src[p], applied in ASCENDING p[dim]
 * for each destination element -- the order of the sequential aten CPU kernel, so fp
 * results are bit-identical to it. self/out contiguous; index/src strided. bf16/f16
 * tensors accumulate in fp32 and round once (as aten CPU does). Wide matrices run on
 * shared-memory strip / row kernels without scratch; tall, narrow or strided geometries
 * are grouped by destination first and need scratch (counters, segment storage): ask
 * b200_scatter_add_scratch_bytes with the same arguments and pass at least that much. */
int64_t b200_scatter_add_scratch_bytes(const void* self, const void* index, const void* src,
                                       const void* out, int ndim, const int64_t* self_shape,
                                       const int64_t* index_shape, const int64_t* index_strides,
                                       const int64_t* src_strides, int dim, int dtype);
int b200_scatter_add(const void* self, const void* index, const void* src, void* out, int ndim,
                     const int64_t* self_shape, const int64_t* index_shape,
                     const int64_t* index_strides, const int64_t* src_strides, int dim,
                     int dtype, void* scratch, int64_t scratch_bytes, uint32_t* status,
                     void* stream);

/* aten.embedding_dense_backward.default(grad_output, indices, num_weights, padding_idx,
 * scale_grad_by_freq = false) -- the backward neighbour at BackendBench/backends/flag_gems.py:113:
 * out[v, :] = sum of grad[i, :] over the positions i with indices[i] == v, v != padding_idx,
 * added in ascending i in fp32 and rounded once (reproducible: no floating-point atomics).
 * grad is [n_indices, row_len], out [num_weights, row_len], both contiguous. */
int64_t b200_embedding_backward_scratch_bytes(int64_t n_indices, int64_t num_weights);
int b200_embedding_backward(const void* grad, const void* indices, void* out, int64_t n_indices,
                            int64_t num_weights, int64_t row_len, int64_t padding_idx, int dtype,
                            int idx_dtype, void* scratch, int64_t scratch_bytes, uint32_t* status,
                            void* stream);

/* ------------------------------------------------------------------ contraction
 * aten.mm.default, aten.addmm.default, aten.bmm.default (eval.py:100-102):
 *   C[b] = alpha * A[b] @ B[b] + beta * bias      (fp32 accumulate, one rounding)
 * A is [batch, M, K] with element strides (sAb, sAm, sAk); B is [batch, K, N] with
 * (sBb, sBk, sBn); C is contiguous [batch, M, N]; bias (may be NULL) has strides
 * (sbias_m, sbias_n), 0 = broadcast. bf16/f16 operands with 16-byte-aligned unit-stride
 * layouts run on tcgen05 tensor cores (TMA-fed, TMEM accumulators); everything else
 * (fp32, odd strides) runs on the CUDA-core kernel. `status` as above (bounded waits). */
int b200_gemm(const void* A, const void* B, const void* bias, void* C, int64_t batch, int64_t M,
              int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk, int64_t sBb,
              int64_t sBk, int64_t sBn, int64_t sbias_m, int64_t sbias_n, double alpha,
              double beta, int dtype, uint32_t* status, void* stream);
/* 1 when the arguments above would take the tcgen05 path, 0 for the CUDA-core path. */
int b200_gemm_uses_tensor_cores(int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb,
                                int64_t sAm, int64_t sAk, int64_t sBb, int64_t sBk, int64_t sBn,
                                int dtype, const void* A, const void* B, const void* C);

/* Failure-detection probe of the tcgen05 kernel's bounded waits (no counterpart in the
 * reference, whose only failure path is a worker that dies on a CUDA error,
 * multiprocessing_eval.py:130-138): runs the tensor-core kernel on row-major bf16/f16
 * A [M, K], B [K, N] with the producer WITHHOLDING the first K slab of every CTA's first
 * tile and with every mbarrier wait limited to `wait_limit_us` (50 .. 100000). Nothing can
 * complete that tile, so the waits run out: the kernel ORs B200_DEV_WAIT_TIMEOUT into
 * *status, frees its tensor memory and returns by itself within a few limits; C is left
 * undefined. The context stays usable and the next b200_gemm is unaffected. Returns
 * B200_EALIGN when the operands would not take the tensor-core path. */
int b200_gemm_wait_probe(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                         int dtype, int64_t wait_limit_us, uint32_t* status, void* stream);

/* The same contraction for fp32 operands on the tensor cores: A and B are split once into
 * three bf16 planes each (x = x1 + x2 + x3 to within 2^-25), written to caller scratch, and
 * the six plane products that matter at fp32 resolution are accumulated in fp32 by the
 * tcgen05 kernel. The result agrees with an fp32 product to a few units in the last place
 * of the accumulated magnitude; it pays off when M*N*K is large (the split is one extra
 * pass over A and B). Operands holding an infinity or a NaN are detected on the device and
 * that product is computed by the CUDA-core kernel instead (fp32 special-value semantics).
 * Any operand strides; C contiguous fp32; bias fp32. Scratch size from
 * b200_gemm_f32_scratch_bytes. (The reference has one matmul per dtype: eval.py:100-102.) */
int64_t b200_gemm_f32_scratch_bytes(int64_t batch, int64_t M, int64_t N, int64_t K);
int b200_gemm_f32(const void* A, const void* B, const void* bias, void* C, int64_t batch,
                  int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk,
                  int64_t sBb, int64_t sBk, int64_t sBn, int64_t sbias_m, int64_t sbias_n,
                  double alpha, double beta, void* scratch, int64_t scratch_bytes,
                  uint32_t* status, void* stream);

/* Small 16-bit products (at most 148 tiles of 64 x 64, K <= 256, at most 2^26 multiply-adds,
 * both operands with one unit stride and base / other strides on the 16-byte grid) are served
 * by a four-warp mma.sync kernel with cp.async staging instead of the tcgen05 kernel, whose
 * set-up alone takes about 5 us. b200_gemm_prefers_small tells a caller whether b200_gemm
 * will go that way.
 * b200_gemm_small_path(0) switches the path off process-wide (1 on again) and returns the
 * previous setting -- for comparisons and for testing the larger kernels on small shapes. */
int b200_gemm_prefers_small(const void* A, const void* B, int64_t batch, int64_t M, int64_t N,
                            int64_t K, int64_t sAb, int64_t sAm, int64_t sAk, int64_t sBb, int64_t sBk,
                            int64_t sBn, int dtype);
int b200_gemm_small_path(int enable);

/* A 16-bit product with a long contraction and a C of a few tiles (batch 1, at most a quarter
 * of the SMs' worth of 128 x 256 tiles, K >= 1536, K divisible by 8 x the number of ranges):
 * the contraction is cut into up to 32 ranges that run as separate CTAs of the tensor-core
 * kernel and leave fp32 partial products in caller scratch; a second kernel adds them in a
 * fixed order, applies alpha / beta / bias and rounds once (deterministic, no atomics).
 * b200_gemm_splitk_scratch_bytes returns the scratch the call needs, 0 when the product does
 * not qualify; b200_gemm_splitk then behaves exactly like b200_gemm. (No counterpart in the
 * reference, which leaves the choice to cuBLAS: eval.py:100-102.) */
int64_t b200_gemm_splitk_scratch_bytes(const void* A, const void* B, const void* C, int64_t batch,
                                       int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm,
                                       int64_t sAk, int64_t sBb, int64_t sBk, int64_t sBn, int dtype);
int b200_gemm_splitk(const void* A, const void* B, const void* bias, void* C, int64_t batch,
                     int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk,
                     int64_t sBb, int64_t sBk, int64_t sBn, int64_t sbias_m, int64_t sbias_n,
                     double alpha, double beta, int dtype, void* scratch, int64_t scratch_bytes,
                     uint32_t* status, void* stream);

/* ------------------------------------------------------------- evaluation path */

/* One pass replacing BackendBench/eval.py:68-90 (`allclose`: torch.testing.assert_close
 * with equal_nan=True) and BackendBench/utils.py:185-242 (`compute_errors`) for one
 * pair of same-shape contiguous tensors. Accumulates into a 32-byte device record:
 *   uint64 mismatches; float max_abs; float max_rel; uint32 nan_seen; uint32 pad[3]
 * mismatch rule: !(ref == res || (isnan both) || |ref-res| <= atol + rtol*|res|).
 * max_rel uses |ref-res| / (|ref| + 1e-10) after conversion to fp32.
 * If `reset` is non-zero the record is zeroed (on the stream) first. */
typedef struct {
  uint64_t mismatches;
  float max_abs;
  float max_rel;
  uint32_t nan_seen;
  uint32_t pad[3];
} b200_close_record;
int b200_allclose(const void* ref, const void* res, int64_t n, int dtype, double rtol,
                  double atol, b200_close_record* record, int reset, void* stream);

/* Evict L2 between timed repetitions: overwrite `bytes` of caller scratch (> L2 size). */
int b200_l2_flush(void* scratch, int64_t bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200OPS_H */
