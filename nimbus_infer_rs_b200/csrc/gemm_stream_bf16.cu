// The decode step's matrix product with a bfloat16 result: the second of the two translation
// units that instantiate the kernel of gemm_stream.cuh (gemm_stream.cu plans the product and
// holds the entry points and the kernels with a 32-bit result).
#include "gemm_stream.cuh"

int nb_gemm_stream_launch_bf16(const void* plan, const void* X, int x_is_f32, const float* gamma,
                               const float* beta, float eps, const void* W, const float* bias,
                               const float* residual, void* out, int M, int N, int K, int act,
                               cudaStream_t stream) {
  const StreamPlan& p = *static_cast<const StreamPlan*>(plan);
  const bool ln = gamma != nullptr;
#define NB_OUT(TX_, LN_) \
  return launch_vpt<TX_, LN_, bf16>(p, X, gamma, beta, eps, W, bias, residual, out, M, N, K, act, stream)
  if (x_is_f32) { if (ln) { NB_OUT(float, true); } else { NB_OUT(float, false); } }
  NB_OUT(bf16, false);
#undef NB_OUT
}

int nb_gemm_stream_bf16_set_wait_budget(long long cycles) { return set_wait_budget(cycles); }
