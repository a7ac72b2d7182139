// Shared declarations of the sm_100a kernel library.
//
// Every exported launcher is `extern "C"`, takes raw device pointers plus the CUDA
// stream to launch on, and returns 0 or an error code; the text of the last error of
// the calling thread is available through nb_last_error().  Nothing in this library
// allocates device memory: callers pass inputs, outputs and scratch.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define NB_EXPORT extern "C" __attribute__((visibility("default")))

// Element types of tensors handed to launchers.
enum NbDType : int { NB_F32 = 0, NB_BF16 = 1 };
// Activation applied in a matrix product's epilogue.
enum NbAct : int { NB_ACT_NONE = 0, NB_ACT_GELU_TANH = 1, NB_ACT_GELU_ERF = 2 };

// Error codes above the range of cudaError_t.
#define NB_ERR_BAD_ARG 10001
#define NB_ERR_UNSUPPORTED 10002
#define NB_ERR_DEVICE_FLAG 10003

void nb_set_error(const char* fmt, ...);

#define NB_REQUIRE(cond, code, ...)                                                     \
  do {                                                                                  \
    if (!(cond)) {                                                                      \
      nb_set_error(__VA_ARGS__);                                                        \
      return (code);                                                                    \
    }                                                                                   \
  } while (0)

#define NB_CHECK_LAUNCH(name)                                                           \
  do {                                                                                  \
    cudaError_t e__ = cudaGetLastError();                                               \
    if (e__ != cudaSuccess) {                                                           \
      nb_set_error("%s: launch failed: %s", (name), cudaGetErrorString(e__));           \
      return (int)e__;                                                                  \
    }                                                                                   \
  } while (0)

#define NB_CUDA(call)                                                                   \
  do {                                                                                  \
    cudaError_t e__ = (call);                                                           \
    if (e__ != cudaSuccess) {                                                           \
      nb_set_error("%s: %s", #call, cudaGetErrorString(e__));                           \
      return (int)e__;                                                                  \
    }                                                                                   \
  } while (0)

// ---------------------------------------------------------------------------------
// Error words: a kernel whose bounded wait ran out says so in a word of pinned host memory
// that is mapped into the device's address space (one word per kernel family, see below).
// The kernel writes it with a plain store and a system-wide fence before it ends, so a host
// that has waited for the stream reads it with a plain load: no copy, no extra
// synchronisation.  nb_error_words() allocates the page on first use (host memory, never
// device memory) and returns nullptr if that fails; kernels given nullptr still give up their
// waits and return, they only cannot say so.
// ---------------------------------------------------------------------------------
enum NbErrorWord : int { NB_ERRW_GEMM_TCGEN05 = 0, NB_ERRW_ATTENTION_PREFILL_TC = 1, NB_ERRW_PROBE = 2, NB_ERRW_GEMM_STREAM = 3, NB_ERRW_GEMM_TC_ROWS = 4, NB_ERRW_COUNT = 16 };
int* nb_error_words();

__device__ __forceinline__ void nb_report_timeout(int* err_word) {
  if (err_word != nullptr) {
    *reinterpret_cast<volatile int*>(err_word) = 1;
    __threadfence_system();
  }
}

// ---------------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched through nb_launch with overlap enabled
// may start while the kernel before it in the stream is still running; it must execute
// nb_grid_dependency_wait() before it reads anything that kernel wrote or writes anything at
// all, and it must do so in every CTA, also in one that has nothing to do: a grid that ended
// without waiting would let its own successor run ahead of the kernel before it.
//
// Every kernel of this library calls nb_launch_dependents() only AFTER its own wait.  A kernel
// therefore starts at the earliest when its predecessor's wait is over, i.e. when everything
// before the predecessor is complete: before its own wait a kernel may read constants
// (weights, biases) and anything written by kernels two or more places ahead of it in the
// stream (the cache of earlier steps, the batch layout), but nothing its direct predecessor
// writes.
//
// A pointer to anything that a kernel of the same step writes (activations, logits, the batch
// layout, the cache) must not be `const __restrict__` in such a kernel: loads through one are
// "invariant" to the compiler, which may then move them in front of the wait, whatever the
// asm statement's memory clobber says -- the kernel reads the rows of the step before.  (It
// happened to the decode attention's query loads, in some builds and not in others, and
// showed only in replayed graphs, where kernels follow each other closely enough to overlap.)
// Constants (weights, biases, a norm's scale and shift) keep the qualifier.  Where the trigger sits after the wait is a matter of speed: the products and the
// decode attention give it once their own loads are on their way.  Without the launch
// attribute both instructions do nothing.
// ---------------------------------------------------------------------------------
bool nb_overlap_enabled();

__device__ __forceinline__ void nb_grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
}
__device__ __forceinline__ void nb_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t nb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = nb_overlap_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same, with the grid cut into thread-block clusters of `cluster_x` CTAs along x
// (grid.x must be a multiple of it).
template <typename... KArgs, typename... Args>
inline cudaError_t nb_launch_clusters(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, int cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = nb_overlap_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---------------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------------
__device__ __forceinline__ float nb_to_f32(float v) { return v; }
__device__ __forceinline__ float nb_to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T nb_from_f32(float v);
template <>
__device__ __forceinline__ float nb_from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 nb_from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// GELU, tanh form: 0.5 x (1 + tanh(0.79788456 (x + 0.044715 x^3)))  (src/ops.rs:21-24)
__device__ __forceinline__ float nb_gelu_tanh(float x) {
  const float c = 0.7978845608028654f;
  return 0.5f * x * (1.0f + tanhf(c * (x + 0.044715f * x * x * x)));
}
// GELU, exact form: 0.5 x (1 + erf(x / sqrt 2))
__device__ __forceinline__ float nb_gelu_erf(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.7071067811865476f));
}
// The tanh form again, written as x * sigmoid(2u) = x / (1 + exp(-2u)) with the hardware
// exponential and reciprocal: a few ulp of fp32 from the line above at a quarter of the
// instructions.  Used in the epilogues of the bf16 kernels, whose results are rounded to
// bf16 (or added to an fp32 stream) anyway; the 32-bit path keeps tanhf.
__device__ __forceinline__ float nb_gelu_tanh_fast(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return __fdividef(x, 1.0f + __expf(-2.0f * u));
}
__device__ __forceinline__ float nb_apply_act_fast(float x, int act) {
  if (act == NB_ACT_GELU_TANH) return nb_gelu_tanh_fast(x);
  if (act == NB_ACT_GELU_ERF) return nb_gelu_erf(x);
  return x;
}
__device__ __forceinline__ float nb_apply_act(float x, int act) {
  if (act == NB_ACT_GELU_TANH) return nb_gelu_tanh(x);
  if (act == NB_ACT_GELU_ERF) return nb_gelu_erf(x);
  return x;
}

__device__ __forceinline__ float nb_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float nb_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum / max for blocks of up to 1024 threads; `red` holds 32 floats.
__device__ __forceinline__ float nb_block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = nb_warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? red[lane] : 0.0f;
  return nb_warp_sum(t);
}
__device__ __forceinline__ float nb_block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = nb_warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? red[lane] : -INFINITY;
  return nb_warp_max(t);
}

// The paged key/value store of one layer: pages of `page` tokens, each
// [n_kv_heads][page][head_dim]; a sequence's pages are listed in its row of the block table.
struct NbPagedKV {
  void* k;                  // [n_pages][n_kv_heads][page][head_dim]
  void* v;
  const int* block_table;   // [n_slots][max_pages]
  int max_pages;
  int page;                 // tokens per page
  int n_kv_heads;
  int head_dim;
};
