/*
 * oracle_ops.c -- TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C, single-threaded CPU restatement of the sixteen operators and of the
 * harness's comparison arithmetic, used only by tests/, __graft_entry__.smoke() and
 * bench.py's CPU-baseline leg as the checker for the CUDA kernels. Nothing in the
 * product path may call it.
 *
 * Where the algorithm lives: the reference (meta-pytorch/BackendBench) computes nothing
 * itself; its reference results are `op(*args, **kwargs)` with op = torch.ops.aten.<op>
 * (BackendBench/eval.py:100, via AtenBackend, BackendBench/backends/aten.py:10-18). The
 * arithmetic is therefore PyTorch ATen, a third-party dependency that is not vendored
 * in the reference tree (pyproject.toml:20, unpinned; the build image has torch
 * 2.11.0+cu128). Each function below restates the published semantics of one aten
 * overload and names the reference call site it stands behind. The restatement is
 * pinned by tests/golden/ (vectors produced by running the reference harness over aten
 * CPU, tests/golden/make_golden.py): integer/index results and scatter_add must match
 * those bit for bit, floating results within the tolerances written in the tests.
 *
 * Floating inputs arrive as fp32 arrays (bf16/f16 tensors are widened by the Python
 * wrapper, exactly); results are produced in fp32 (after double-precision accumulation)
 * and rounded to the tensor dtype by the wrapper with round-to-nearest-even, which is
 * what aten's opmath convention does: compute in fp32, round once.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- rounding helpers (the wrapper calls these to narrow fp32 results) ------------ */

/* fp32 -> bf16 bits, round to nearest even, NaN stays NaN (quiet). */
uint16_t oracle_f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
float oracle_bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
void oracle_round_bf16(const float* x, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = oracle_f32_to_bf16(x[i]);
}
void oracle_round_f16(const float* x, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    _Float16 h = (_Float16)x[i];
    memcpy(&out[i], &h, 2);
  }
}
void oracle_widen_bf16(const uint16_t* x, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = oracle_bf16_to_f32(x[i]);
}
void oracle_widen_f16(const uint16_t* x, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    _Float16 h;
    memcpy(&h, &x[i], 2);
    out[i] = (float)h;
  }
}

/* ---- elementwise (same-shape contiguous; the wrapper materialises broadcasts) ----- */

/* aten.relu.default: clamp_min(x, 0); NaN propagates. eval.py:100. */
void oracle_relu(const float* x, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = (x[i] != x[i]) ? x[i] : (x[i] > 0.f ? x[i] : 0.f);
}
/* aten.add.Tensor: self + alpha * other in fp32 opmath. eval.py:100. */
void oracle_add(const float* a, const float* b, float* out, int64_t n, float alpha) {
  for (int64_t i = 0; i < n; ++i) out[i] = (float)((double)a[i] + (double)alpha * (double)b[i]);
}
/* aten.mul.Tensor. eval.py:100. */
void oracle_mul(const float* a, const float* b, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = a[i] * b[i];
}
/* aten.where.self: byte-wise select, elem_size bytes per element. eval.py:100. */
void oracle_where(const uint8_t* cond, const uint8_t* x, const uint8_t* y, uint8_t* out, int64_t n, int elem_size) {
  for (int64_t i = 0; i < n; ++i) memcpy(out + i * elem_size, (cond[i] ? x : y) + i * elem_size, (size_t)elem_size);
}

/* ---- row operators on a contiguous [outer, dim, inner] view ---------------------- */

/* aten._softmax.default / aten._log_softmax.default (dim, half_to_float): the max is
 * taken ignoring NaN (a NaN input then poisons the sum through exp), inf - inf = NaN as
 * in IEEE arithmetic. eval.py:100. */
void oracle_softmax(const float* x, float* out, int64_t outer, int64_t dim, int64_t inner, int is_log) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      const float* p = x + o * dim * inner + i;
      float* q = out + o * dim * inner + i;
      float m = -INFINITY;
      for (int64_t k = 0; k < dim; ++k) {
        const float v = p[k * inner];
        if (v > m) m = v; /* NaN compares false: skipped */
      }
      double s = 0.0;
      for (int64_t k = 0; k < dim; ++k) s += exp((double)(p[k * inner] - m));
      const double ls = log(s);
      for (int64_t k = 0; k < dim; ++k) {
        const double d = (double)(p[k * inner] - m);
        q[k * inner] = is_log ? (float)(d - ls) : (float)(exp(d) / s);
      }
    }
}

/* aten._softmax_backward_data.default / aten._log_softmax_backward_data.default
 * (grad_output, output, dim, input_dtype) -- the backward neighbours listed at
 * BackendBench/backends/flag_gems.py:196,233; evaluated through eval.py:100 like any op.
 *   softmax:     gin = (g - sum(g * y)) * y        log_softmax: gin = g - exp(y) * sum(g) */
void oracle_softmax_backward(const float* g, const float* y, float* out, int64_t outer, int64_t dim, int64_t inner, int is_log) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      const int64_t base = o * dim * inner + i;
      double s = 0.0;
      for (int64_t k = 0; k < dim; ++k) s += is_log ? (double)g[base + k * inner] : (double)g[base + k * inner] * (double)y[base + k * inner];
      for (int64_t k = 0; k < dim; ++k) {
        const double gv = g[base + k * inner], yv = y[base + k * inner];
        out[base + k * inner] = (float)(is_log ? gv - exp(yv) * s : (gv - s) * yv);
      }
    }
}

/* aten.sum.dim_IntList over `dim` of [outer, dim, inner]; empty dim sums to 0. eval.py:100. */
void oracle_sum(const float* x, float* out, int64_t outer, int64_t dim, int64_t inner) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      double s = 0.0;
      for (int64_t k = 0; k < dim; ++k) s += (double)x[(o * dim + k) * inner + i];
      out[o * inner + i] = (float)s;
    }
}

/* aten.native_layer_norm.default -> (out, mean, rstd): biased variance, rstd =
 * 1/sqrt(var + eps), out = (x - mean) * rstd * w + b; w, b may be NULL. A row holding a
 * NaN or an infinity gets NaN statistics and a NaN output row: aten's running (Welford)
 * moments turn inf into NaN as soon as another element follows it (only an infinity in
 * the very last position leaves mean = inf there). eval.py:100; output triple as
 * BackendBench/backends/flag_gems.py:19-31. */
void oracle_layer_norm(const float* x, const float* w, const float* b, float* y, float* mean, float* rstd, int64_t rows, int64_t cols, double eps) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* p = x + r * cols;
    double s = 0.0;
    for (int64_t c = 0; c < cols; ++c) s += (double)p[c];
    double mu = s / (double)cols;
    if (!isfinite(mu)) mu = NAN;
    double q = 0.0;
    for (int64_t c = 0; c < cols; ++c) {
      const double d = (double)p[c] - mu;
      q += d * d;
    }
    const double rs = 1.0 / sqrt(q / (double)cols + eps);
    mean[r] = (float)mu;
    rstd[r] = (float)rs;
    for (int64_t c = 0; c < cols; ++c) {
      double v = ((double)p[c] - mu) * rs;
      if (w) v *= (double)w[c];
      if (b) v += (double)b[c];
      y[r * cols + c] = (float)v;
    }
  }
}

/* aten.embedding_dense_backward.default (grad_output, indices, num_weights, padding_idx,
 * scale_grad_by_freq = false) -- BackendBench/backends/flag_gems.py:113; evaluated through
 * eval.py:100. Rows are added in ascending position, fp32 accumulation (the caller rounds
 * once). Returns the number of out-of-range indices (skipped). */
int64_t oracle_embedding_backward(const float* grad, const int64_t* idx, float* out, int64_t n, int64_t num_weights, int64_t row_len, int64_t padding_idx) {
  int64_t bad = 0;
  for (int64_t k = 0; k < num_weights * row_len; ++k) out[k] = 0.f;
  for (int64_t i = 0; i < n; ++i) {
    const int64_t v = idx[i];
    if (v == padding_idx) continue;
    if (v < 0 || v >= num_weights) { ++bad; continue; }
    for (int64_t c = 0; c < row_len; ++c) out[v * row_len + c] += grad[i * row_len + c];
  }
  return bad;
}

/* aten.native_layer_norm_backward.default (grad_out, input, normalized_shape, mean, rstd,
 * weight, bias, output_mask) -- BackendBench/backends/flag_gems.py:140; evaluated through
 * eval.py:100. w may be NULL; dx / dw / db may be NULL (masked outputs). */
void oracle_layer_norm_backward(const float* dy, const float* x, const float* mean, const float* rstd, const float* w, float* dx, float* dw, float* db, int64_t rows, int64_t cols) {
  if (dw) for (int64_t c = 0; c < cols; ++c) dw[c] = 0.f;
  if (db) for (int64_t c = 0; c < cols; ++c) db[c] = 0.f;
  double* aw = dw ? (double*)calloc((size_t)(cols > 0 ? cols : 1), sizeof(double)) : NULL;
  double* ab = db ? (double*)calloc((size_t)(cols > 0 ? cols : 1), sizeof(double)) : NULL;
  for (int64_t r = 0; r < rows; ++r) {
    const double mu = mean[r], rs = rstd[r];
    double s1 = 0.0, s2 = 0.0;
    for (int64_t c = 0; c < cols; ++c) {
      const double g = dy[r * cols + c], xhat = ((double)x[r * cols + c] - mu) * rs, gy = g * (w ? (double)w[c] : 1.0);
      s1 += gy;
      s2 += gy * xhat;
      if (aw) aw[c] += g * xhat;
      if (ab) ab[c] += g;
    }
    if (dx) {
      const double c1 = s1 / (double)cols, c2 = s2 / (double)cols;
      for (int64_t c = 0; c < cols; ++c) {
        const double xhat = ((double)x[r * cols + c] - mu) * rs, gy = (double)dy[r * cols + c] * (w ? (double)w[c] : 1.0);
        dx[r * cols + c] = (float)(rs * (gy - c1 - xhat * c2));
      }
    }
  }
  if (aw) { for (int64_t c = 0; c < cols; ++c) dw[c] = (float)aw[c]; free(aw); }
  if (ab) { for (int64_t c = 0; c < cols; ++c) db[c] = (float)ab[c]; free(ab); }
}

/* aten.argmax.default along `dim` of [outer, dim, inner]: first index of the maximum,
 * NaN counts as the maximum (the first NaN wins). eval.py:100. */
void oracle_argmax(const float* x, int64_t* out, int64_t outer, int64_t dim, int64_t inner) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      int64_t best = 0;
      float bv = x[o * dim * inner + i];
      for (int64_t k = 1; k < dim && bv == bv; ++k) {
        const float v = x[(o * dim + k) * inner + i];
        if (v != v || v > bv) { bv = v; best = k; }
      }
      out[o * inner + i] = best;
    }
}

/* ---- indexing (bit copies) --------------------------------------------------------- */

/* aten.embedding.default / aten.index_select.default on [outer, dim_size, inner_bytes]:
 * out[o, k, :] = x[o, idx[k], :]. Returns the number of out-of-range indices (aten
 * raises IndexError for those; their rows are zero-filled here). eval.py:100. */
int64_t oracle_index_select(const uint8_t* x, const int64_t* idx, uint8_t* out, int64_t outer, int64_t dim_size, int64_t inner_bytes, int64_t n_idx) {
  int64_t bad = 0;
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t k = 0; k < n_idx; ++k) {
      uint8_t* d = out + (o * n_idx + k) * inner_bytes;
      if (idx[k] < 0 || idx[k] >= dim_size) {
        memset(d, 0, (size_t)inner_bytes);
        ++bad;
      } else {
        memcpy(d, x + (o * dim_size + idx[k]) * inner_bytes, (size_t)inner_bytes);
      }
    }
  return bad;
}

/* aten.gather.default on N-d tensors: out[p] = self[p with p[dim] := index[p]].
 * `self_strides` in elements, index/out contiguous with `index_shape`. eval.py:100. */
int64_t oracle_gather(const uint8_t* self, const int64_t* index, uint8_t* out, int ndim, const int64_t* index_shape, const int64_t* self_strides, int64_t self_dim_size,
                      int dim, int elem_size) {
  int64_t n = 1, bad = 0;
  for (int d = 0; d < ndim; ++d) n *= index_shape[d];
  for (int64_t p = 0; p < n; ++p) {
    int64_t lin = p, so = 0;
    for (int d = ndim - 1; d >= 0; --d) {
      const int64_t r = lin % index_shape[d];
      lin /= index_shape[d];
      if (d != dim) so += r * self_strides[d];
    }
    const int64_t k = index[p];
    if (k < 0 || k >= self_dim_size) {
      memset(out + p * elem_size, 0, (size_t)elem_size);
      ++bad;
    } else {
      memcpy(out + p * elem_size, self + (so + k * self_strides[dim]) * elem_size, (size_t)elem_size);
    }
  }
  return bad;
}

/* aten.scatter_add.default: out = self; then, walking index in row-major order (so the
 * `dim` coordinate ascends for every fixed remainder), out[p with p[dim] := index[p]] +=
 * src[p], one fp32 addition per contribution. 16-bit tensors accumulate in an fp32 copy
 * of self and are rounded once at the end (the wrapper narrows `out`), which is what the
 * sequential aten CPU kernel does with its opmath buffer -- so results are bit-comparable
 * for fp32, bf16 and f16 alike. eval.py:100. */
int64_t oracle_scatter_add(float* out, const int64_t* index, const float* src, int ndim, const int64_t* self_shape, const int64_t* index_shape, const int64_t* src_shape, int dim) {
  int64_t n = 1, bad = 0;
  int64_t self_strides[16], src_strides[16];
  for (int d = 0; d < ndim; ++d) n *= index_shape[d];
  int64_t a = 1, b = 1;
  for (int d = ndim - 1; d >= 0; --d) {
    self_strides[d] = a;
    a *= self_shape[d];
    src_strides[d] = b;
    b *= src_shape[d];
  }
  for (int64_t p = 0; p < n; ++p) {
    int64_t lin = p, so = 0, ro = 0;
    for (int d = ndim - 1; d >= 0; --d) {
      const int64_t r = lin % index_shape[d];
      lin /= index_shape[d];
      if (d != dim) so += r * self_strides[d];
      ro += r * src_strides[d];
    }
    const int64_t k = index[p];
    if (k < 0 || k >= self_shape[dim]) { ++bad; continue; }
    out[so + k * self_strides[dim]] += src[ro];
  }
  return bad;
}

/* ---- contraction ------------------------------------------------------------------- */

/* aten.mm / aten.addmm / aten.bmm: C[b] = alpha * A[b] @ B[b] + beta * bias, contiguous
 * row-major operands, double accumulation (the tests allow for aten's fp32 accumulation
 * order); beta == 0 ignores bias entirely. eval.py:100. */
void oracle_gemm(const float* A, const float* B, const float* bias, float* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sbias_m, int64_t sbias_n, double alpha,
                 double beta) {
  double* acc = (double*)malloc((size_t)(N > 0 ? N : 1) * sizeof(double));
  for (int64_t b = 0; b < batch; ++b)
    for (int64_t m = 0; m < M; ++m) {
      for (int64_t n = 0; n < N; ++n) acc[n] = 0.0;
      for (int64_t k = 0; k < K; ++k) {
        const double a = (double)A[(b * M + m) * K + k];
        const float* brow = B + (b * K + k) * N;
        for (int64_t n = 0; n < N; ++n) acc[n] += a * (double)brow[n];
      }
      for (int64_t n = 0; n < N; ++n) {
        double r = alpha * acc[n];
        if (bias && beta != 0.0) r += beta * (double)bias[m * sbias_m + n * sbias_n];
        C[(b * M + m) * N + n] = (float)r;
      }
    }
  free(acc);
}

/* ---- the harness's comparison ------------------------------------------------------ */

/* BackendBench/eval.py:68-90 (`allclose`: torch.testing.assert_close(ref, res,
 * equal_nan=True, atol, rtol)) and BackendBench/utils.py:185-242 (`compute_errors`) for
 * one pair of fp32 arrays. out[0] = number of mismatching elements, out[1] = max abs
 * error, out[2] = max rel error (|ref-res| / (|ref| + 1e-10)); the maxima are NaN as soon
 * as one difference is NaN, like `.abs().max()`. */
void oracle_compare(const float* ref, const float* res, int64_t n, double rtol, double atol, double* out) {
  double bad = 0, mabs = 0, mrel = 0;
  int nan_seen = 0;
  for (int64_t i = 0; i < n; ++i) {
    const float r = ref[i], s = res[i];
    const int rn = r != r, sn = s != s;
    const double diff = fabs((double)r - (double)s);
    const int close = (r == s) || (rn && sn) || (!rn && !sn && isfinite(diff) && diff <= atol + rtol * fabs((double)s));
    if (!close) bad += 1;
    const float fd = fabsf(r - s);
    if (fd != fd) nan_seen = 1;
    else {
      if (fd > mabs) mabs = fd;
      const float rel = fd / (fabsf(r) + 1e-10f);
      if (rel > mrel) mrel = rel;
    }
  }
  out[0] = bad;
  out[1] = nan_seen ? NAN : mabs;
  out[2] = nan_seen ? NAN : mrel;
}
