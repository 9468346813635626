// mm / addmm / bmm entry point: picks the tcgen05 tensor-core kernel when the operands
// qualify (bf16/f16, TMA-compatible layout) and the CUDA-core kernel otherwise.
#include <atomic>

#include "b200_common.cuh"

namespace b200 {
int gemm_simt_dispatch(const void* A, const void* B, const void* bias, void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk,
                       int64_t sBb, int64_t sBk, int64_t sBn, int64_t sbm, int64_t sbn, double alpha, double beta, int dtype, cudaStream_t st, const uint32_t* gate = nullptr);
bool gemm_tc_eligible(int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk, int64_t sBb, int64_t sBk, int64_t sBn, int dtype,
                      const void* A, const void* B, const void* C);
int gemm_tc_dispatch(const void* A, const void* B, const void* bias, void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk,
                     int64_t sBb, int64_t sBk, int64_t sBn, int64_t sbm, int64_t sbn, double alpha, double beta, int dtype, uint32_t* status, cudaStream_t st,
                     uint64_t wait_probe_limit_ns = 0, bool allow_pair = true);

bool gemm_mma_small_preferred(const void* A, const void* B, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk, int64_t sBb, int64_t sBk, int64_t sBn,
                              int dtype);
int gemm_mma_small_dispatch(const void* A, const void* B, const void* bias, void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk, int64_t sBb,
                            int64_t sBk, int64_t sBn, int64_t sbm, int64_t sbn, double alpha, double beta, int dtype, cudaStream_t st);
int64_t gemm_tc_splitk_scratch_bytes(int64_t batch, int64_t M, int64_t N, int64_t K);
int gemm_tc_splitk_dispatch(const void* A, const void* B, const void* bias, void* C, int64_t M, int64_t N, int64_t K, int64_t sAm, int64_t sAk, int64_t sBk, int64_t sBn, int64_t sbm,
                            int64_t sbn, double alpha, double beta, int dtype, void* scratch, int64_t scratch_bytes, uint32_t* status, cudaStream_t st);

int64_t gemm_f32_split_scratch_bytes(int64_t batch, int64_t M, int64_t N, int64_t K);
bool gemm_f32_split_eligible(int64_t batch, int64_t M, int64_t N, int64_t K);
int gemm_f32_split_dispatch(const void* A, const void* B, const void* bias, void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk, int64_t sBb,
                            int64_t sBk, int64_t sBn, int64_t sbm, int64_t sbn, double alpha, double beta, void* scratch, int64_t scratch_bytes, uint32_t* status, cudaStream_t st);

// 1: small 16-bit products take the mma.sync kernel (the default); 0: they go where they went
// without it (tcgen05 or CUDA cores) -- how the two are compared and the larger kernels tested
// on small shapes.
static std::atomic<int> g_small_path{1};

__global__ void fill_bias_only(void* C, const void* bias, int64_t batch, int64_t M, int64_t N, int64_t sbm, int64_t sbn, float beta, int dt) {
  const int64_t total = batch * M * N;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t n = i % N, m = (i / N) % M;
    const float r = (bias && beta != 0.f) ? beta * load_as_f32(bias, m * sbm + n * sbn, dt) : 0.f;
    store_from_f32(C, i, dt, r);
  }
}
}  // namespace b200

using namespace b200;

extern "C" int b200_gemm_uses_tensor_cores(int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk, int64_t sBb, int64_t sBk, int64_t sBn,
                                           int dtype, const void* A, const void* B, const void* C) {
  return gemm_tc_eligible(batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, dtype, A, B, C) ? 1 : 0;
}

extern "C" int b200_gemm(const void* A, const void* B, const void* bias, void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk,
                         int64_t sBb, int64_t sBk, int64_t sBn, int64_t sbm, int64_t sbn, double alpha, double beta, int dtype, uint32_t* status, void* stream) {
  if (batch < 0 || M < 0 || N < 0 || K < 0) return B200_EINVAL;
  if (!is_float_dtype(dtype)) return B200_EDTYPE;
  if (batch == 0 || M == 0 || N == 0) return B200_OK;
  if (!C) return B200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (K == 0) {  // empty contraction: the product is zero, only beta * bias remains
    int64_t blocks = (batch * M * N + 255) / 256;
    if (blocks > kNumSMs * 16) blocks = kNumSMs * 16;
    fill_bias_only<<<static_cast<int>(blocks), 256, 0, st>>>(C, bias, batch, M, N, sbm, sbn, static_cast<float>(beta), dtype);
    return check_launch();
  }
  if (!A || !B) return B200_EINVAL;
  if (g_small_path.load(std::memory_order_relaxed) && gemm_mma_small_preferred(A, B, batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, dtype))
    return gemm_mma_small_dispatch(A, B, bias, C, batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn, alpha, beta, dtype, st);
  if (gemm_tc_eligible(batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, dtype, A, B, C))
    return gemm_tc_dispatch(A, B, bias, C, batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn, alpha, beta, dtype, status, st);
  return gemm_simt_dispatch(A, B, bias, C, batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn, alpha, beta, dtype, st);
}

extern "C" int b200_gemm_wait_probe(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int dtype, int64_t wait_limit_us, uint32_t* status, void* stream) {
  if (M < 1 || N < 1 || K < 1 || !A || !B || !C || !status) return B200_EINVAL;
  if (wait_limit_us < 50 || wait_limit_us > 100000) return B200_EINVAL;  // 50 us .. 0.1 s
  // row-major A [M, K] and B [K, N], the tensor-core path or nothing
  if (!gemm_tc_eligible(1, M, N, K, 0, K, 1, 0, N, 1, dtype, A, B, C)) return B200_EALIGN;
  return gemm_tc_dispatch(A, B, nullptr, C, 1, M, N, K, 0, K, 1, 0, N, 1, 0, 0, 1.0, 0.0, dtype, status, static_cast<cudaStream_t>(stream), static_cast<uint64_t>(wait_limit_us) * 1000ull);
}

extern "C" int64_t b200_gemm_f32_scratch_bytes(int64_t batch, int64_t M, int64_t N, int64_t K) {
  if (!gemm_f32_split_eligible(batch, M, N, K)) return 0;
  return gemm_f32_split_scratch_bytes(batch, M, N, K);
}

extern "C" int b200_gemm_f32(const void* A, const void* B, const void* bias, void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk,
                             int64_t sBb, int64_t sBk, int64_t sBn, int64_t sbm, int64_t sbn, double alpha, double beta, void* scratch, int64_t scratch_bytes, uint32_t* status,
                             void* stream) {
  if (batch < 0 || M < 0 || N < 0 || K < 0) return B200_EINVAL;
  if (batch == 0 || M == 0 || N == 0) return B200_OK;
  if (K == 0 || !gemm_f32_split_eligible(batch, M, N, K)) return b200_gemm(A, B, bias, C, batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn, alpha, beta, B200_F32, status, stream);
  if (!A || !B || !C) return B200_EINVAL;
  return gemm_f32_split_dispatch(A, B, bias, C, batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn, alpha, beta, scratch, scratch_bytes, status, static_cast<cudaStream_t>(stream));
}

extern "C" int64_t b200_gemm_splitk_scratch_bytes(const void* A, const void* B, const void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk,
                                                  int64_t sBb, int64_t sBk, int64_t sBn, int dtype) {
  if (batch != 1 || M < 1 || N < 1 || K < 1) return 0;
  if (!gemm_tc_eligible(batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, dtype, A, B, C)) return 0;
  return gemm_tc_splitk_scratch_bytes(batch, M, N, K);
}

extern "C" int b200_gemm_splitk(const void* A, const void* B, const void* bias, void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk,
                                int64_t sBb, int64_t sBk, int64_t sBn, int64_t sbm, int64_t sbn, double alpha, double beta, int dtype, void* scratch, int64_t scratch_bytes,
                                uint32_t* status, void* stream) {
  // anything the split does not serve (see b200_gemm_splitk_scratch_bytes) is an ordinary product
  if (b200_gemm_splitk_scratch_bytes(A, B, C, batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, dtype) == 0)
    return b200_gemm(A, B, bias, C, batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, sbm, sbn, alpha, beta, dtype, status, stream);
  return gemm_tc_splitk_dispatch(A, B, bias, C, M, N, K, sAm, sAk, sBk, sBn, sbm, sbn, alpha, beta, dtype, scratch, scratch_bytes, status, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_gemm_small_path(int enable) { return g_small_path.exchange(enable ? 1 : 0); }

extern "C" int b200_gemm_prefers_small(const void* A, const void* B, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t sAb, int64_t sAm, int64_t sAk, int64_t sBb, int64_t sBk,
                                       int64_t sBn, int dtype) {
  return (g_small_path.load(std::memory_order_relaxed) && gemm_mma_small_preferred(A, B, batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, dtype)) ? 1 : 0;
}
