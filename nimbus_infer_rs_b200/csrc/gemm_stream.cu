// Matrix products of a decode step (at most 16 rows), bf16 weights:
// out[M,N] = act(norm?(X)[M,K] * W[N,K]^T + bias) (+ residual).
//
// Such a product is a stream of weights from HBM, and in a small model it is one link of a
// long chain of dependent kernels: what counts is that the weights are already on the SM when
// the rows arrive.  So the weights do not pass through registers.  A CTA owns a few groups of
// 8 output columns; before it waits for the kernel in front of it (programmatic dependent
// launch), one warp asks for its weight rows with TMA tile loads (boxes of the batch's rows x 64
// columns, completion counted on an mbarrier) into a ring of shared-memory stages, and lets the
// kernel behind it start.  With few registers and little shared memory per CTA the CTAs of several
// kernels of the chain sit on an SM at the same time, each with its weights landing while the
// kernels before it still compute: HBM keeps streaming across kernel boundaries.  After the
// wait the rows are staged (LayerNorm applied on the way: statistics in fp32, two passes,
// src/ops.rs:32-40; the norm's weight and bias were fetched before the wait, they are
// constants), the warps multiply with mma.sync (bf16 in, fp32 accumulate) from shared memory,
// partial sums of warps that split K meet in shared memory, and the epilogue adds bias,
// activation and residual.
//
// A work item is (batch of G column groups, chunk of K); a CTA walks its items through the
// ring: a product with few columns has one item per CTA, all of it requested before the wait;
// the output head (50,257 columns) is a long walk with the ring refilled as stages drain.
//
// Before the wait a kernel touches constants only (weights, biases, norm vectors); it lets its
// successor start right after its own wait, as every kernel of the library does (common.cuh).
//
// Every wait on an mbarrier is bounded by a clock budget; a wait that runs out raises an error
// word, the CTA skips its stores, gives its copies time to land and returns.
//
// Reference analogue: Mat::gemv_into (src/model.rs:65-86), one dot product per output.
#include "gemm_stream.cuh"

// 1 if nb_gemm_stream takes this product (bf16 weights; `ln`: with the LayerNorm of the rows
// folded in).  Otherwise the caller uses the other product kernels.
NB_EXPORT int nb_gemm_stream_supported(int M, int N, int K, int ln) {
  return plan_stream(M, N, K, ln != 0).ok ? 1 : 0;
}

// How nb_gemm_stream would cut the product, for reports and tests: out[0..12] = groups of 16
// columns per batch, warps along the columns, K per work item, work items per batch, stages, bytes
// between weight rows, elements between staged rows, threads per row of the norm, groups of
// 16 columns, warps, row vectors per thread of the norm, CTAs, bytes of shared memory.  Returns 0 if the
// product is not taken.
NB_EXPORT int nb_gemm_stream_plan(int M, int N, int K, int ln, int* out) {
  const StreamPlan p = plan_stream(M, N, K, ln != 0);
  if (!p.ok) return 0;
  const int v[13] = {p.sh.GB, p.sh.wn, p.sh.n_kbox * 64, p.sh.n_kc, p.sh.S, 128, p.sh.x_stride,
                     p.sh.tpr, p.sh.n16, p.nw, p.vpt, p.grid, (int)p.smem};
  for (int i = 0; i < 13; ++i) out[i] = v[i];
  return 1;
}

// Tuning: the most CTAs a product is cut into (0: one per SM at most, every CTA as many column
// groups as the others).
NB_EXPORT int nb_gemm_stream_tune(int target_ctas) {
  g_target_ctas = target_ctas > 0 ? target_ctas : 0;
  return 0;
}

// Clock cycles a wait of this kernel may take before it gives up (default 4e9).
NB_EXPORT int nb_gemm_stream_set_wait_budget(long long cycles) {
  NB_REQUIRE(cycles >= 0, NB_ERR_BAD_ARG, "wait budget must not be negative");
  const int rc = set_wait_budget(cycles);
  return rc ? rc : nb_gemm_stream_bf16_set_wait_budget(cycles);
}

// M <= 16, bf16 weights [N, K] with K % 8 == 0.  gamma != nullptr asks for LayerNorm of the
// rows first (X must then be fp32); `residual` may alias `out` (fp32).
NB_EXPORT int nb_gemm_stream(const void* X, int x_dtype, const float* gamma, const float* beta,
                             float eps, const void* W, const float* bias, const float* residual,
                             void* out, int out_dtype, int M, int N, int K, int act,
                             cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  const bool ln = gamma != nullptr;
  const StreamPlan p = plan_stream(M, N, K, ln);
  NB_REQUIRE(p.ok, NB_ERR_UNSUPPORTED, "gemm_stream: does not take M=%d N=%d K=%d%s", M, N, K,
             ln ? " with a norm" : "");
  NB_REQUIRE(!ln || x_dtype == NB_F32, NB_ERR_BAD_ARG, "gemm_stream: a fused norm needs fp32 rows");
  NB_REQUIRE((uintptr_t)W % 16 == 0 && (uintptr_t)X % 16 == 0, NB_ERR_UNSUPPORTED,
             "gemm_stream: rows and weights must be 16-byte aligned");
  int rc = 0;
  if (out_dtype != NB_F32) {   // results in bfloat16: the kernels of the other translation unit
    rc = nb_gemm_stream_launch_bf16(&p, X, x_dtype == NB_F32, gamma, beta, eps, W, bias, residual, out, M,
                                    N, K, act, stream);
  } else {
#define NB_OUT(TX_, LN_) \
  rc = launch_vpt<TX_, LN_, float>(p, X, gamma, beta, eps, W, bias, residual, out, M, N, K, act, stream)
    if (x_dtype == NB_F32) { if (ln) { NB_OUT(float, true); } else { NB_OUT(float, false); } }
    else { NB_OUT(bf16, false); }
#undef NB_OUT
  }
  if (rc) return rc;
  NB_CHECK_LAUNCH("gemm_stream");
  return 0;
}
