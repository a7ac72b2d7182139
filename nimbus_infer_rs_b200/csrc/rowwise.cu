// Row-wise kernels: token+position embedding, LayerNorm, key/value append into the paged
// cache.  One thread block per row; any width.
#include <stdarg.h>

#include "common.cuh"

// ---------------------------------------------------------------------------------
// error text of the calling thread
// ---------------------------------------------------------------------------------
static thread_local char g_error[512] = "";

void nb_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

NB_EXPORT const char* nb_last_error() { return g_error; }

NB_EXPORT int nb_abi_version() { return 3; }

// ---------------------------------------------------------------------------------
// error words (see common.cuh)
// ---------------------------------------------------------------------------------
#include <mutex>
static int* g_error_words = nullptr;
int* nb_error_words() {
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    if (cudaHostAlloc(&p, NB_ERRW_COUNT * sizeof(int), cudaHostAllocPortable | cudaHostAllocMapped) ==
        cudaSuccess) {
      for (int i = 0; i < NB_ERRW_COUNT; ++i) static_cast<volatile int*>(p)[i] = 0;
      g_error_words = static_cast<int*>(p);
    } else {
      (void)cudaGetLastError();
    }
  });
  return g_error_words;
}
// Bit i is set if error word i is raised.  No synchronisation: the caller has waited for the
// work it asks about.  `clear` != 0 lowers the words that were read as raised.
NB_EXPORT int nb_device_errors(int clear) {
  volatile int* w = nb_error_words();
  if (w == nullptr) return 0;
  int mask = 0;
  for (int i = 0; i < NB_ERRW_COUNT; ++i) {
    if (w[i] != 0) {
      mask |= 1 << i;
      if (clear) w[i] = 0;
    }
  }
  return mask;
}

// Whether kernels are launched so that they may overlap the tail of their predecessor.
static int g_overlap = 0;
bool nb_overlap_enabled() { return g_overlap != 0; }
NB_EXPORT void nb_set_overlap(int on) { g_overlap = on; }
NB_EXPORT int nb_get_overlap() { return g_overlap; }

// ---------------------------------------------------------------------------------
// x[r] = wte[token[r]] + wpe[pos[r]]   (src/model.rs:285-295), fp32 result.
// A negative token marks a padding row: it is written as zeros.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void embed_pos_kernel(const int* tokens, const int* pos,
                                 const T* __restrict__ wte, const T* __restrict__ wpe,
                                 float* out, int d) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int r = blockIdx.x;
  const int tok = tokens[r];
  float* o = out + (size_t)r * d;
  if (tok < 0) {
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = 0.0f;
    return;
  }
  const T* e = wte + (size_t)tok * d;
  if (wpe != nullptr) {
    const T* p = wpe + (size_t)pos[r] * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = nb_to_f32(e[i]) + nb_to_f32(p[i]);
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = nb_to_f32(e[i]);
  }
}

NB_EXPORT int nb_embed_pos(const int* tokens, const int* pos, const void* wte, const void* wpe,
                           int table_dtype, float* out, int n_rows, int d, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(n_rows > 0 && d > 0, NB_ERR_BAD_ARG, "embed_pos: bad sizes rows=%d d=%d", n_rows, d);
  const int threads = d >= 256 ? 256 : (d >= 128 ? 128 : 64);
  if (table_dtype == NB_F32)
    NB_CUDA(nb_launch(embed_pos_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, tokens, pos,
                      (const float*)wte, (const float*)wpe, out, d));
  else if (table_dtype == NB_BF16)
    NB_CUDA(nb_launch(embed_pos_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream,
                      tokens, pos, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, out, d));
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "embed_pos: unknown table dtype %d", table_dtype);
  NB_CHECK_LAUNCH("embed_pos");
  return 0;
}

// ---------------------------------------------------------------------------------
// LayerNorm of fp32 rows (src/ops.rs:32-40): mean, biased variance of (x - mean), both in
// fp32 and in two passes; y = (x - mean) / sqrt(var + eps) * gamma + beta.
// `rows` (optional) selects the source row of each output row; a negative entry gives zeros.
// The row is kept in shared memory between the passes.
// ---------------------------------------------------------------------------------
template <typename TOut>
__global__ void layernorm_kernel(const float* x, const int* rows,
                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                 TOut* out, int d, float eps) {
  extern __shared__ float row[];
  __shared__ float red[32];
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  TOut* o = out + (size_t)r * d;
  if (src < 0) {
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = nb_from_f32<TOut>(0.0f);
    return;
  }
  const float* xr = x + (size_t)src * d;
  float s = 0.0f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = xr[i];
    row[i] = v;
    s += v;
  }
  const float mean = nb_block_sum(s, red) / (float)d;
  float q = 0.0f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float c = row[i] - mean;
    q += c * c;
  }
  const float var = nb_block_sum(q, red) / (float)d;
  const float inv = 1.0f / sqrtf(var + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float y = (row[i] - mean) * inv * gamma[i];
    if (beta) y += beta[i];
    o[i] = nb_from_f32<TOut>(y);
  }
}

// The same, one warp per row with the row held in registers (one trip to memory): widths that
// are a multiple of 4 up to 128 * VN.  EARLY: scale and shift are fetched into registers
// before the wait on the kernel in front (they are constants), which takes their trip to
// memory out of a decode step's chain (batch 64: 0.98 -> 0.93 ms a step on GPT-2 124M, 4.26
// -> 3.72 ms on XL); with thousands of rows the registers cost more CTAs per SM than the trip
// is worth (a 2,048-token prefill: 1.15 -> 1.25 ms), so those fetch them where they are used.
template <typename TOut, int VN, bool EARLY>
__global__ void __launch_bounds__(128)
layernorm_warp_kernel(const float* x, const int* rows,
                      const float* __restrict__ gamma, const float* __restrict__ beta,
                      TOut* out, int n_rows, int d, float eps) {
  const int lane = threadIdx.x & 31;
  float4 gm[EARLY ? VN : 1], bt[EARLY ? VN : 1];
  if constexpr (EARLY) {
#pragma unroll
    for (int i = 0; i < VN; ++i) {
      const int k = lane * 4 + i * 128;
      gm[i] = k < d ? *reinterpret_cast<const float4*>(gamma + k) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      bt[i] = (beta && k < d) ? *reinterpret_cast<const float4*>(beta + k)
                              : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
  }
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const int src = rows ? rows[r] : r;
  TOut* o = out + (size_t)r * d;
  float4 v[VN];
  const float* xr = x + (size_t)(src < 0 ? 0 : src) * d;
#pragma unroll
  for (int i = 0; i < VN; ++i) {
    const int k = lane * 4 + i * 128;
    v[i] = (src >= 0 && k < d) ? *reinterpret_cast<const float4*>(xr + k)
                               : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  }
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < VN; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  const float mean = nb_warp_sum(s) / (float)d;
  float q = 0.0f;
#pragma unroll
  for (int i = 0; i < VN; ++i) {
    if (lane * 4 + i * 128 < d) {
      const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, e = v[i].w - mean;
      q += (a * a + b * b) + (c * c + e * e);
    }
  }
  const float inv = 1.0f / sqrtf(nb_warp_sum(q) / (float)d + eps);
#pragma unroll
  for (int i = 0; i < VN; ++i) {
    const int k = lane * 4 + i * 128;
    if (k >= d) continue;
    float4 y = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (src >= 0) {
      float4 g4, b4;
      if constexpr (EARLY) {
        g4 = gm[i];
        b4 = bt[i];
      } else {
        g4 = *reinterpret_cast<const float4*>(gamma + k);
        b4 = beta ? *reinterpret_cast<const float4*>(beta + k) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
      y.x = (v[i].x - mean) * inv * g4.x + b4.x;
      y.y = (v[i].y - mean) * inv * g4.y + b4.y;
      y.z = (v[i].z - mean) * inv * g4.z + b4.z;
      y.w = (v[i].w - mean) * inv * g4.w + b4.w;
    }
    if constexpr (sizeof(TOut) == 4) {
      *reinterpret_cast<float4*>(o + k) = y;
    } else {
      uint2 pk;
      *reinterpret_cast<__nv_bfloat162*>(&pk.x) = __floats2bfloat162_rn(y.x, y.y);
      *reinterpret_cast<__nv_bfloat162*>(&pk.y) = __floats2bfloat162_rn(y.z, y.w);
      *reinterpret_cast<uint2*>(o + k) = pk;
    }
  }
}

template <typename TOut>
int launch_layernorm_warp(const float* x, const int* rows, const float* gamma, const float* beta,
                          void* out, int n_rows, int d, float eps, cudaStream_t stream) {
  const dim3 grid((n_rows + 3) / 4), block(128);
  const bool early = n_rows <= 512;   // one CTA per SM or so: registers are free
#define NB_LN(VN_)                                                                              \
  do {                                                                                          \
    if (early)                                                                                  \
      NB_CUDA(nb_launch(layernorm_warp_kernel<TOut, VN_, true>, grid, block, 0, stream, x, rows, \
                        gamma, beta, (TOut*)out, n_rows, d, eps));                              \
    else                                                                                        \
      NB_CUDA(nb_launch(layernorm_warp_kernel<TOut, VN_, false>, grid, block, 0, stream, x, rows, \
                        gamma, beta, (TOut*)out, n_rows, d, eps));                              \
  } while (0)
  if (d <= 128 * 2) NB_LN(2);
  else if (d <= 128 * 8) NB_LN(8);
  else NB_LN(16);
#undef NB_LN
  return 0;
}

NB_EXPORT int nb_layernorm(const float* x, const int* rows, const float* gamma, const float* beta,
                           void* out, int out_dtype, int n_rows, int d, float eps,
                           cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(n_rows > 0 && d > 0, NB_ERR_BAD_ARG, "layernorm: bad sizes rows=%d d=%d", n_rows, d);
  if (d % 4 == 0 && d <= 128 * 16 && (uintptr_t)x % 16 == 0 && (uintptr_t)gamma % 16 == 0 &&
      (uintptr_t)beta % 16 == 0 && (uintptr_t)out % 16 == 0 &&
      (out_dtype == NB_F32 || out_dtype == NB_BF16)) {
    const int rc = out_dtype == NB_F32
                       ? launch_layernorm_warp<float>(x, rows, gamma, beta, out, n_rows, d, eps, stream)
                       : launch_layernorm_warp<__nv_bfloat16>(x, rows, gamma, beta, out, n_rows, d,
                                                              eps, stream);
    if (rc) return rc;
    NB_CHECK_LAUNCH("layernorm");
    return 0;
  }
  const size_t smem = (size_t)d * sizeof(float);
  NB_REQUIRE(smem <= 200 * 1024, NB_ERR_UNSUPPORTED,
             "layernorm: width %d needs %zu bytes of shared memory (limit 204800)", d, smem);
  const int threads = d >= 1024 ? 256 : (d >= 256 ? 128 : 64);
  if (out_dtype == NB_F32) {
    if (smem > 48 * 1024)
      NB_CUDA(cudaFuncSetAttribute(layernorm_kernel<float>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    NB_CUDA(nb_launch(layernorm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, x, rows,
                      gamma, beta, (float*)out, d, eps));
  } else if (out_dtype == NB_BF16) {
    if (smem > 48 * 1024)
      NB_CUDA(cudaFuncSetAttribute(layernorm_kernel<__nv_bfloat16>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    NB_CUDA(nb_launch(layernorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), smem, stream, x,
                      rows, gamma, beta, (__nv_bfloat16*)out, d, eps));
  } else {
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "layernorm: unknown output dtype %d", out_dtype);
  }
  NB_CHECK_LAUNCH("layernorm");
  return 0;
}

// ---------------------------------------------------------------------------------
// Append this step's keys and values to the paged cache (src/cache.rs:44-57 writes rows
// P..P+T of every head).  Row r of `src` holds [.. | K: n_kv_heads*head_dim | V: same ..]
// starting at column k_col / v_col; it goes to token `pos[r]` of sequence slot `slot[r]`.
// Rows with a negative slot are padding and are skipped.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ src, int src_stride, int k_col, int v_col,
                                 const int* row_slot, const int* row_pos,
                                 NbPagedKV kv) {
  const int r = blockIdx.x;
  const int slot = row_slot[r];
  if (slot < 0) return;
  const int pos = row_pos[r];
  const int page_id = kv.block_table[(size_t)slot * kv.max_pages + pos / kv.page];
  const int in_page = pos % kv.page;
  const int width = kv.n_kv_heads * kv.head_dim;
  const T* srow = src + (size_t)r * src_stride;
  T* kdst = (T*)kv.k;
  T* vdst = (T*)kv.v;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const int h = i / kv.head_dim, c = i - h * kv.head_dim;
    const size_t o =
        (((size_t)page_id * kv.n_kv_heads + h) * kv.page + in_page) * kv.head_dim + c;
    kdst[o] = srow[k_col + i];
    vdst[o] = srow[v_col + i];
  }
}

// The same in 16-byte pieces (head size, columns and pitch multiples of 16 bytes): a warp takes
// a row at a time, the lanes its pieces; a block of 8 warps walks over rows.
template <typename T>
__global__ void __launch_bounds__(256)
kv_append_vec_kernel(const T* __restrict__ src, int src_stride, int k_col, int v_col,
                     const int* row_slot, const int* row_pos,
                     NbPagedKV kv, int n_rows) {
  constexpr int E = 16 / sizeof(T);              // elements per piece
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pieces_per_head = kv.head_dim / E;
  const int pieces = kv.n_kv_heads * pieces_per_head;   // of K, and as many of V
  for (int r = blockIdx.x * 8 + warp; r < n_rows; r += gridDim.x * 8) {
    const int slot = row_slot[r];
    if (slot < 0) continue;
    const int pos = row_pos[r];
    const int page_id = kv.block_table[(size_t)slot * kv.max_pages + pos / kv.page];
    const int in_page = pos % kv.page;
    const T* srow = src + (size_t)r * src_stride;
    for (int i = lane; i < 2 * pieces; i += 32) {
      const bool is_v = i >= pieces;
      const int p = is_v ? i - pieces : i;
      const int h = p / pieces_per_head, c = (p - h * pieces_per_head) * E;
      const size_t o = (((size_t)page_id * kv.n_kv_heads + h) * kv.page + in_page) * kv.head_dim + c;
      const uint4 val = *reinterpret_cast<const uint4*>(srow + (is_v ? v_col : k_col) + p * E);
      *reinterpret_cast<uint4*>((is_v ? (T*)kv.v : (T*)kv.k) + o) = val;
    }
  }
}

NB_EXPORT int nb_kv_append(const void* src, int dtype, int src_stride, int k_col, int v_col,
                           const int* row_slot, const int* row_pos, void* k_cache, void* v_cache,
                           const int* block_table, int max_pages, int page, int n_kv_heads,
                           int head_dim, int n_rows, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NbPagedKV kv{k_cache, v_cache, block_table, max_pages, page, n_kv_heads, head_dim};
  const int width = n_kv_heads * head_dim;
  const int threads = width >= 256 ? 256 : (width >= 128 ? 128 : 64);
  const int esize = dtype == NB_F32 ? 4 : 2, e16 = 16 / esize;
  const bool vec = (dtype == NB_F32 || dtype == NB_BF16) && head_dim % e16 == 0 &&
                   src_stride % e16 == 0 && k_col % e16 == 0 && v_col % e16 == 0 &&
                   (uintptr_t)src % 16 == 0 && (uintptr_t)k_cache % 16 == 0 &&
                   (uintptr_t)v_cache % 16 == 0;
  if (vec) {
    const int blocks = (n_rows + 7) / 8 < 148 * 8 ? (n_rows + 7) / 8 : 148 * 8;
    if (dtype == NB_F32)
      kv_append_vec_kernel<float><<<blocks, 256, 0, stream>>>(
          (const float*)src, src_stride, k_col, v_col, row_slot, row_pos, kv, n_rows);
    else
      kv_append_vec_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
          (const __nv_bfloat16*)src, src_stride, k_col, v_col, row_slot, row_pos, kv, n_rows);
    NB_CHECK_LAUNCH("kv_append");
    return 0;
  }
  if (dtype == NB_F32)
    kv_append_kernel<float><<<n_rows, threads, 0, stream>>>((const float*)src, src_stride, k_col,
                                                            v_col, row_slot, row_pos, kv);
  else if (dtype == NB_BF16)
    kv_append_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>(
        (const __nv_bfloat16*)src, src_stride, k_col, v_col, row_slot, row_pos, kv);
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "kv_append: unknown dtype %d", dtype);
  NB_CHECK_LAUNCH("kv_append");
  return 0;
}

// ---------------------------------------------------------------------------------
// Between two decode steps on the device: the sampled token becomes the next input and the
// position of every live row moves on by one.  Rows with a negative slot are padding.
// ---------------------------------------------------------------------------------
__global__ void advance_decode_kernel(int* tokens, const int* next,
                                      int* row_pos, const int* row_slot,
                                      int n) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (row_slot[i] >= 0) {
    tokens[i] = next[i];
    row_pos[i] += 1;
  } else {
    tokens[i] = -1;
  }
}

NB_EXPORT int nb_advance_decode(int* tokens, const int* next, int* row_pos, const int* row_slot,
                                int n, cudaStream_t stream) {
  if (n == 0) return 0;
  NB_CUDA(nb_launch(advance_decode_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, tokens, next,
                    row_pos, row_slot, n));
  NB_CHECK_LAUNCH("advance_decode");
  return 0;
}
