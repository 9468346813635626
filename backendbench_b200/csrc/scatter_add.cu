// scatter_add with the aten CPU kernel's summation order (bit-identical fp results).
//
// For every destination element the contributions src[p] are added one after another in
// ascending p[dim], starting from self -- exactly what the sequential CPU loop does.
// Atomics cannot reproduce that order, so ordering is made structural:
//
//   strip kernel (2-D, dim 0, fp32): a CTA owns a strip of 8 output columns and keeps
//     the whole strip [rows x 8] in shared memory (column-major, so random destination
//     rows spread over the banks). Source rows arrive in tiles of 128 rows through a
//     cp.async double buffer (64-byte index segments, 32-byte value segments). Warp w
//     owns column w of the strip and walks the tile 32 source rows at a time, in
//     order; lanes that target the same destination row are found with
//     __match_any_sync and applied in lane (= source-row) order. Different columns
//     never interact, different tiles are separated by a CTA barrier. HBM traffic is
//     the algorithmic minimum: self, index, src read once, out written once.
//
//   line kernel (everything else): one thread per "line" (all coordinates but `dim`
//     fixed) applies its contributions sequentially in global memory, after a copy of
//     self. bf16/f16 tensors accumulate in an fp32 copy of self held in caller scratch
//     and are rounded once at the end, as the aten CPU kernel does with its fp32 buffer.
#include <cuda_pipeline.h>

#include "b200_common.cuh"

namespace b200 {

constexpr int kStripCols = 8;
constexpr int kTileRows = 128;
constexpr int kStripThreads = 256;  // 8 warps = 8 columns

struct StripSmem {
  // out strip first (rows * 8 floats), then two tiles of indices and values
  static size_t bytes(int64_t rows) {
    return static_cast<size_t>(rows) * kStripCols * sizeof(float) + 2 * kTileRows * kStripCols * (sizeof(int64_t) + sizeof(float));
  }
};

__global__ void __launch_bounds__(kStripThreads, 1)
scatter_add_strip_f32(const float* __restrict__ self, const int64_t* __restrict__ index, const float* __restrict__ src, float* __restrict__ out,
                      int64_t rows, int64_t cols, int64_t idx_rows, int64_t idx_cols, int64_t idx_pitch, int64_t src_pitch, uint32_t* status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int64_t* idx_s = reinterpret_cast<int64_t*>(smem_raw);                                  // [2][kTileRows][8]
  float* src_s = reinterpret_cast<float*>(idx_s + 2 * kTileRows * kStripCols);            // [2][kTileRows][8]
  float* strip = src_s + 2 * kTileRows * kStripCols;                                      // [8][rows]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t nstrips = cols / kStripCols;
  const int64_t ntiles = (idx_rows + kTileRows - 1) / kTileRows;

  for (int64_t sidx = blockIdx.x; sidx < nstrips; sidx += gridDim.x) {
    const int64_t j0 = sidx * kStripCols;
    // ---- stage self[:, j0:j0+8] column-major into shared memory (two 16-byte loads per row)
    for (int64_t q = tid; q < rows * 2; q += kStripThreads) {
      const int64_t r = q >> 1;
      const int h = static_cast<int>(q & 1);
      const uint4 v = __ldcs(reinterpret_cast<const uint4*>(self + r * cols + j0 + 4 * h));
      strip[(4 * h + 0) * rows + r] = __uint_as_float(v.x);
      strip[(4 * h + 1) * rows + r] = __uint_as_float(v.y);
      strip[(4 * h + 2) * rows + r] = __uint_as_float(v.z);
      strip[(4 * h + 3) * rows + r] = __uint_as_float(v.w);
    }
    const bool active = j0 < idx_cols;  // strips right of the index matrix are pure copies
    if (active) {
      auto issue_tile = [&](int64_t tile, int buf) {
        // 128 rows x (4 index chunks + 2 value chunks) of 16 bytes = 768 chunks, 3 per thread
        const int64_t i0 = tile * kTileRows;
        for (int c = tid; c < kTileRows * 6; c += kStripThreads) {
          const int r = c / 6, k = c - r * 6;
          const int64_t i = i0 + r;
          if (i < idx_rows) {
            if (k < 4) __pipeline_memcpy_async(idx_s + (buf * kTileRows + r) * kStripCols + 2 * k, index + i * idx_pitch + j0 + 2 * k, 16);
            else __pipeline_memcpy_async(src_s + (buf * kTileRows + r) * kStripCols + 4 * (k - 4), src + i * src_pitch + j0 + 4 * (k - 4), 16);
          }
        }
        __pipeline_commit();
      };
      issue_tile(0, 0);
      for (int64_t tile = 0; tile < ntiles; ++tile) {
        const int buf = static_cast<int>(tile & 1);
        if (tile + 1 < ntiles) {
          issue_tile(tile + 1, buf ^ 1);
          __pipeline_wait_prior(1);
        } else {
          __pipeline_wait_prior(0);
        }
        __syncthreads();  // tile `buf` landed; also orders the strip staging before first use
        float* col = strip + static_cast<int64_t>(warp) * rows;
        const int64_t i0 = tile * kTileRows;
#pragma unroll 1
        for (int sub = 0; sub < kTileRows / 32; ++sub) {
          const int r = sub * 32 + lane;
          const bool valid = i0 + r < idx_rows;
          int64_t key = valid ? idx_s[(buf * kTileRows + r) * kStripCols + warp] : -1 - lane;
          const float v = valid ? src_s[(buf * kTileRows + r) * kStripCols + warp] : 0.f;
          bool apply = valid;
          if (valid && (key < 0 || key >= rows)) {
            if (status) atomicOr(status, B200_DEV_INDEX_OOB);
            apply = false;
            key = -1 - lane;  // unique, never matches another lane
          }
          const unsigned peers = __match_any_sync(0xffffffffu, key);
          const int rank = __popc(peers & ((1u << lane) - 1u));
          unsigned pending = __ballot_sync(0xffffffffu, apply);
          for (int turn = 0; pending; ++turn) {
            if (apply && rank == turn) {
              col[key] += v;
              apply = false;
            }
            __syncwarp();
            pending = __ballot_sync(0xffffffffu, apply);
          }
        }
        __syncthreads();  // everyone done with tile `buf` before it is refilled
      }
    } else {
      __syncthreads();
    }
    // ---- write the strip back
    for (int64_t q = tid; q < rows * 2; q += kStripThreads) {
      const int64_t r = q >> 1;
      const int h = static_cast<int>(q & 1);
      uint4 v;
      v.x = __float_as_uint(strip[(4 * h + 0) * rows + r]);
      v.y = __float_as_uint(strip[(4 * h + 1) * rows + r]);
      v.z = __float_as_uint(strip[(4 * h + 2) * rows + r]);
      v.w = __float_as_uint(strip[(4 * h + 3) * rows + r]);
      __stcs(reinterpret_cast<uint4*>(out + r * cols + j0 + 4 * h), v);
    }
    __syncthreads();  // strip is rewritten by the next iteration
  }
}

// ------------------------------------------------------------------ generic line kernel
struct ScatterArgs {
  int ndim, dim;
  int64_t nlines, dim_len, self_dim_size;
  int64_t shape[B200_MAX_DIMS];  // index shape with shape[dim] forced to 1
  int64_t out_stride[B200_MAX_DIMS], idx_stride[B200_MAX_DIMS], src_stride[B200_MAX_DIMS];
};

template <typename T>
__global__ void __launch_bounds__(128) scatter_add_lines(float* __restrict__ out, const int64_t* __restrict__ index, const T* __restrict__ src, ScatterArgs A, uint32_t* status) {
  const int64_t line = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (line >= A.nlines) return;
  int64_t lin = line, oo = 0, io = 0, so = 0;
  for (int d = A.ndim - 1; d >= 0; --d) {
    const int64_t q = lin / A.shape[d], r = lin - q * A.shape[d];
    oo += r * A.out_stride[d];
    io += r * A.idx_stride[d];
    so += r * A.src_stride[d];
    lin = q;
  }
  const int64_t os = A.out_stride[A.dim], is = A.idx_stride[A.dim], ss = A.src_stride[A.dim];
  for (int64_t k = 0; k < A.dim_len; ++k) {
    const int64_t key = index[io + k * is];
    if (key < 0 || key >= A.self_dim_size) {
      if (status) atomicOr(status, B200_DEV_INDEX_OOB);
      continue;
    }
    out[oo + key * os] += to_f32(src[so + k * ss]);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_scatter_add(const void* self, const void* index, const void* src, void* out, int ndim, const int64_t* self_shape, const int64_t* index_shape,
                                const int64_t* index_strides, const int64_t* src_strides, int dim, int dtype, void* scratch, int64_t scratch_bytes, uint32_t* status, void* stream) {
  if (ndim < 1 || ndim > B200_MAX_DIMS || dim < 0 || dim >= ndim || !self_shape || !index_shape || !index_strides || !src_strides) return B200_EINVAL;
  if (!is_float_dtype(dtype)) return B200_EDTYPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t n_self = numel_of(ndim, self_shape);
  const int64_t n_idx = numel_of(ndim, index_shape);
  for (int d = 0; d < ndim; ++d)
    if (self_shape[d] < 0 || index_shape[d] < 0 || (d != dim && index_shape[d] > self_shape[d])) return B200_EINVAL;
  if (n_self == 0) return B200_OK;
  if (!self || !out) return B200_EINVAL;
  const int es = dtype_size(dtype);

  // ---- strip kernel eligibility
  if (n_idx > 0 && ndim == 2 && dim == 0 && dtype == B200_F32 && index && src) {
    const int64_t rows = self_shape[0], cols = self_shape[1];
    const size_t smem = StripSmem::bytes(rows);
    const bool fits = smem <= 200 * 1024;
    const bool shape_ok = cols % kStripCols == 0 && index_shape[1] % kStripCols == 0;
    const bool stride_ok = index_strides[1] == 1 && src_strides[1] == 1 && index_strides[0] % 2 == 0 && src_strides[0] % 4 == 0;
    if (fits && shape_ok && stride_ok && aligned16(self) && aligned16(out) && aligned16(index) && aligned16(src)) {
      // per device and cheap, so set on every call rather than cached per process
      const cudaError_t ae = cudaFuncSetAttribute(scatter_add_strip_f32, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (ae != cudaSuccess) { set_last_cuda_error(ae); return B200_ELAUNCH; }
      const int64_t nstrips = cols / kStripCols;
      const int grid = static_cast<int>(nstrips < 4LL * kNumSMs ? nstrips : 4LL * kNumSMs);
      scatter_add_strip_f32<<<grid, kStripThreads, smem, st>>>(static_cast<const float*>(self), static_cast<const int64_t*>(index), static_cast<const float*>(src), static_cast<float*>(out),
                                                                rows, cols, index_shape[0], index_shape[1], index_strides[0], src_strides[0], status);
      return check_launch();
    }
  }

  // ---- generic: acc = fp32(self), ordered lines on acc, out = round(acc)
  const bool wide = dtype == B200_F32;
  float* acc = wide ? static_cast<float*>(out) : static_cast<float*>(scratch);
  if (!wide && (!scratch || scratch_bytes < n_self * 4)) return B200_ESCRATCH;
  if (wide) {
    if (out != self) {
      const cudaError_t ce = cudaMemcpyAsync(out, self, static_cast<size_t>(n_self) * es, cudaMemcpyDeviceToDevice, st);
      if (ce != cudaSuccess) { set_last_cuda_error(ce); return B200_ELAUNCH; }
    }
  } else {
    const int64_t one = 1;
    if (int rc = b200_copy_strided(self, acc, 1, &n_self, &one, dtype, B200_F32, stream)) return rc;
  }
  if (n_idx > 0) {
    if (!index || !src) return B200_EINVAL;
    ScatterArgs A;
    A.ndim = ndim;
    A.dim = dim;
    A.dim_len = index_shape[dim];
    A.self_dim_size = self_shape[dim];
    A.nlines = 1;
    int64_t st_out = 1;
    for (int d = ndim - 1; d >= 0; --d) {
      A.shape[d] = d == dim ? 1 : index_shape[d];
      A.nlines *= A.shape[d];
      A.out_stride[d] = st_out;
      st_out *= self_shape[d];
      A.idx_stride[d] = index_strides[d];
      A.src_stride[d] = src_strides[d];
    }
    const int g = grid_for(A.nlines, 128);
    const int64_t* pi = static_cast<const int64_t*>(index);
    switch (dtype) {
      case B200_F32: scatter_add_lines<float><<<g, 128, 0, st>>>(acc, pi, static_cast<const float*>(src), A, status); break;
      case B200_BF16: scatter_add_lines<__nv_bfloat16><<<g, 128, 0, st>>>(acc, pi, static_cast<const __nv_bfloat16*>(src), A, status); break;
      default: scatter_add_lines<__half><<<g, 128, 0, st>>>(acc, pi, static_cast<const __half*>(src), A, status); break;
    }
    if (int rc = check_launch()) return rc;
  }
  if (!wide) {
    const int64_t one = 1;
    return b200_copy_strided(acc, out, 1, &n_self, &one, B200_F32, dtype, stream);
  }
  return B200_OK;
}
