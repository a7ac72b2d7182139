// Matrix product on the CUDA cores with fp32 multiply-add: out[M,N] = X[M,K] * W[N,K]^T
// with the shared epilogue (bias, GELU, residual add).  This is the whole-model 32-bit
// path (no tensor-core rounding of inputs) and the plain reference path for bf16 inputs:
// inputs are widened to fp32 and every product and sum is an fp32 FMA.
//
// Reference analogue: Mat::gemm_into / gemv_into (src/model.rs:65-133): y[i][j] = dot(x[i],
// Wt[j]) with Wt stored (out, in).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16;
constexpr int THREADS = 256;

template <typename T>
__device__ __forceinline__ void load4(const T* __restrict__ base, int row, int n_rows, int k0,
                                      int K, bool vec_ok, float (&v)[4]) {
  if (row >= n_rows) {
    v[0] = v[1] = v[2] = v[3] = 0.0f;
    return;
  }
  const T* p = base + (size_t)row * K + k0;
  if (vec_ok && k0 + 4 <= K) {
    if constexpr (sizeof(T) == 4) {
      const float4 f = *reinterpret_cast<const float4*>(p);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
      const uint2 u = *reinterpret_cast<const uint2*>(p);
      const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
      const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
      v[0] = __bfloat162float(a.x); v[1] = __bfloat162float(a.y);
      v[2] = __bfloat162float(b.x); v[3] = __bfloat162float(b.y);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = (k0 + i < K) ? nb_to_f32(p[i]) : 0.0f;
  }
}

template <typename TIn, typename TW, typename TOut>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const TIn* __restrict__ X, const TW* __restrict__ W,
                 const float* __restrict__ bias, const float* residual, TOut* out, int M, int N,
                 int K, int act, bool x_vec, bool w_vec) {
  __shared__ float Xs[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;  // each thread loads 4 consecutive k of one row
  const int ty = tid >> 4, tx = tid & 15;         // 16x16 threads, 4x4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  // the next K block is fetched into registers while the current one is multiplied
  float xv[4], wv[4];
  load4<TIn>(X, m0 + lrow, M, lk, K, x_vec, xv);
  load4<TW>(W, n0 + lrow, N, lk, K, w_vec, wv);
  for (int k0 = 0; k0 < K; k0 += BK) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      Xs[lk + i][lrow] = xv[i];
      Ws[lk + i][lrow] = wv[i];
    }
    __syncthreads();
    if (k0 + BK < K) {
      load4<TIn>(X, m0 + lrow, M, k0 + BK + lk, K, x_vec, xv);
      load4<TW>(W, n0 + lrow, N, k0 + BK + lk, K, w_vec, wv);
    }
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&Xs[k][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w};
      const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
  }

  // `residual` may be `out` itself: fetch all of it before the first store, or every load
  // would have to wait for the store before it
  float res[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      res[i][j] = (residual && m < M && n < N) ? residual[(size_t)m * N + n] : 0.0f;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      v = nb_apply_act(v, act);
      out[(size_t)m * N + n] = nb_from_f32<TOut>(v + res[i][j]);
    }
  }
}

template <typename TIn, typename TW, typename TOut>
int launch(const void* X, const void* W, const float* bias, const float* residual, void* out,
           int M, int N, int K, int act, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  // four consecutive elements are fetched with one load when every row start is aligned
  const bool x_vec = (K % 4 == 0) && ((uintptr_t)X % (4 * sizeof(TIn)) == 0);
  const bool w_vec = (K % 4 == 0) && ((uintptr_t)W % (4 * sizeof(TW)) == 0);
  gemm_simt_kernel<TIn, TW, TOut><<<grid, THREADS, 0, stream>>>(
      (const TIn*)X, (const TW*)W, bias, residual, (TOut*)out, M, N, K, act, x_vec, w_vec);
  return 0;
}

}  // namespace

// out = act(X W^T + bias) [+ residual].  `residual` (fp32 [M,N]) may alias `out` when the
// output type is fp32: every element is read and written by the same thread.
NB_EXPORT int nb_gemm_simt(const void* X, int x_dtype, const void* W, int w_dtype,
                           const float* bias, const float* residual, void* out, int out_dtype,
                           int M, int N, int K, int act, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  NB_REQUIRE(M > 0 && N > 0 && K > 0, NB_ERR_BAD_ARG, "gemm_simt: bad sizes M=%d N=%d K=%d", M, N,
             K);
  NB_REQUIRE((M + BM - 1) / BM <= 65535, NB_ERR_UNSUPPORTED, "gemm_simt: M=%d too large", M);
  typedef __nv_bfloat16 bf16;
  const int key = x_dtype * 4 + w_dtype * 2 + out_dtype;
  switch (key) {
    case 0: launch<float, float, float>(X, W, bias, residual, out, M, N, K, act, stream); break;
    case 1: launch<float, float, bf16>(X, W, bias, residual, out, M, N, K, act, stream); break;
    case 2: launch<float, bf16, float>(X, W, bias, residual, out, M, N, K, act, stream); break;
    case 3: launch<float, bf16, bf16>(X, W, bias, residual, out, M, N, K, act, stream); break;
    case 4: launch<bf16, float, float>(X, W, bias, residual, out, M, N, K, act, stream); break;
    case 5: launch<bf16, float, bf16>(X, W, bias, residual, out, M, N, K, act, stream); break;
    case 6: launch<bf16, bf16, float>(X, W, bias, residual, out, M, N, K, act, stream); break;
    case 7: launch<bf16, bf16, bf16>(X, W, bias, residual, out, M, N, K, act, stream); break;
    default:
      NB_REQUIRE(false, NB_ERR_BAD_ARG, "gemm_simt: unknown dtypes x=%d w=%d out=%d", x_dtype,
                 w_dtype, out_dtype);
  }
  NB_CHECK_LAUNCH("gemm_simt");
  return 0;
}
