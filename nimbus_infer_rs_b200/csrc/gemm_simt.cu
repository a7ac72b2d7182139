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

// ---------------------------------------------------------------------------------------
// The same product for large operands (a prompt in the 32-bit path): 128 x 128 output tiles,
// 8 x 8 outputs a thread (as four 4 x 4 corners, so that a warp's shared-memory reads are
// two broadcasts and one unbroken row), K in blocks of 16 through two shared-memory buffers:
// while a block is multiplied the next one is already on its way from memory into registers,
// and goes into the other buffer, so the block costs one barrier.
// ---------------------------------------------------------------------------------------
constexpr int LBM = 128, LBN = 128, LBK = 16, LLD = LBM + 4;

template <typename T>
__device__ __forceinline__ float4 load_quad(const T* __restrict__ base, int row, int n_rows, int k0,
                                            int K, bool vec_ok) {
  float v[4];
  load4<T>(base, row, n_rows, k0, K, vec_ok, v);
  return make_float4(v[0], v[1], v[2], v[3]);
}

template <typename TIn, typename TW, typename TOut>
__global__ void __launch_bounds__(THREADS, 2)
gemm_simt_large_kernel(const TIn* __restrict__ X, const TW* __restrict__ W,
                       const float* __restrict__ bias, const float* residual, TOut* out, int M,
                       int N, int K, int act, bool x_vec, bool w_vec) {
  __shared__ __align__(16) float Xs[2][LBK][LLD];
  __shared__ __align__(16) float Ws[2][LBK][LLD];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * LBM, n0 = blockIdx.x * LBN;
  // loads: a warp takes 32 consecutive rows of one group of four columns of K (its stores into
  // the transposed tile then fall into 32 different banks); two such quads a thread and operand
  const int lrow = tid & 127, lkq = tid >> 7;            // quads lkq and lkq + 2
  const int ty = tid >> 4, tx = tid & 15;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

  float4 xr[2], wr[2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      xr[j] = load_quad<TIn>(X, m0 + lrow, M, k0 + (lkq + 2 * j) * 4, K, x_vec);
      wr[j] = load_quad<TW>(W, n0 + lrow, N, k0 + (lkq + 2 * j) * 4, K, w_vec);
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int k = (lkq + 2 * j) * 4;
      Xs[buf][k][lrow] = xr[j].x; Xs[buf][k + 1][lrow] = xr[j].y;
      Xs[buf][k + 2][lrow] = xr[j].z; Xs[buf][k + 3][lrow] = xr[j].w;
      Ws[buf][k][lrow] = wr[j].x; Ws[buf][k + 1][lrow] = wr[j].y;
      Ws[buf][k + 2][lrow] = wr[j].z; Ws[buf][k + 3][lrow] = wr[j].w;
    }
  };
  fetch(0);
  stash(0);
  __syncthreads();
  const int n_blocks = (K + LBK - 1) / LBK;
  for (int b = 0; b < n_blocks; ++b) {
    const int buf = b & 1;
    if (b + 1 < n_blocks) fetch((b + 1) * LBK);
#pragma unroll
    for (int k = 0; k < LBK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&Xs[buf][k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&Xs[buf][k][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Ws[buf][k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Ws[buf][k][64 + tx * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (b + 1 < n_blocks) stash(buf ^ 1);
    __syncthreads();
  }

  // rows ty*4 + i and 64 + ty*4 + i, columns tx*4 + j and 64 + tx*4 + j.  `residual` may be
  // `out` itself: every element is read and then written by the same thread.
  const bool vec_out = (N % 4 == 0) && sizeof(TOut) == 4 &&
                       ((uintptr_t)out % 16 == 0) && (residual == nullptr || (uintptr_t)residual % 16 == 0);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + (i >> 2) * 64 + ty * 4 + (i & 3);
    if (m >= M) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = n0 + h * 64 + tx * 4;
      if (n >= N) continue;
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[j] = acc[i][h * 4 + j];
        if (bias && n + j < N) v[j] += bias[n + j];
        v[j] = nb_apply_act(v[j], act);
      }
      const size_t o = (size_t)m * N + n;
      if (vec_out && n + 4 <= N) {
        if (residual) {
          const float4 r = *reinterpret_cast<const float4*>(residual + o);
          v[0] += r.x; v[1] += r.y; v[2] += r.z; v[3] += r.w;
        }
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + o) = make_float4(v[0], v[1], v[2], v[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (n + j >= N) continue;
          const float r = residual ? residual[o + j] : 0.0f;
          out[o + j] = nb_from_f32<TOut>(v[j] + r);
        }
      }
    }
  }
}

template <typename TIn, typename TW, typename TOut>
int launch(const void* X, const void* W, const float* bias, const float* residual, void* out,
           int M, int N, int K, int act, cudaStream_t stream) {
  // four consecutive elements are fetched with one load when every row start is aligned
  const bool x_vec = (K % 4 == 0) && ((uintptr_t)X % (4 * sizeof(TIn)) == 0);
  const bool w_vec = (K % 4 == 0) && ((uintptr_t)W % (4 * sizeof(TW)) == 0);
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  // the large tiles when they fill the GPU (two CTAs fit on an SM); fewer of them leave SMs idle,
  // and four times as many small tiles then do better
  if ((long long)((M + LBM - 1) / LBM) * ((N + LBN - 1) / LBN) >= (3 * sms) / 2) {
    dim3 grid((N + LBN - 1) / LBN, (M + LBM - 1) / LBM);
    gemm_simt_large_kernel<TIn, TW, TOut><<<grid, THREADS, 0, stream>>>(
        (const TIn*)X, (const TW*)W, bias, residual, (TOut*)out, M, N, K, act, x_vec, w_vec);
    return 0;
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
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
