// Causal attention of packed query rows over the paged key/value cache, all arithmetic in
// fp32 on the CUDA cores.  It serves prefill and decode alike (a query row at position p of
// its sequence attends to keys 0..p, all of which are in the cache by the time it runs), any
// head size up to 256, any number of heads and key/value groups, and an optional window.
// This is the 32-bit path and the fallback of the bf16 path for shapes that the tensor-core
// kernels refuse.
//
// Reference: src/model.rs:401-422 (score = dot(q,k)*scale for keys 0..P+i, softmax with the
// maximum subtracted src/ops.rs:6-18, weighted sum of values), head h reads key/value head
// h / group (src/model.rs:390).
#include "common.cuh"

namespace {

constexpr int THREADS = 256;
constexpr int CHUNK = 1024;  // keys whose scores are held in shared memory at a time

template <typename T>
__device__ __forceinline__ const T* kv_row(const T* base, const NbPagedKV& kv, int slot, int kvh,
                                           int j) {
  const int page_id = kv.block_table[(size_t)slot * kv.max_pages + j / kv.page];
  return base + (((size_t)page_id * kv.n_kv_heads + kvh) * kv.page + (j % kv.page)) * kv.head_dim;
}

template <typename T, typename TOut>
__global__ void __launch_bounds__(THREADS)
attention_generic_kernel(const T* __restrict__ q, int q_stride, int q_col,
                         const int* __restrict__ row_slot, const int* __restrict__ row_pos,
                         NbPagedKV kv, int group, TOut* __restrict__ out, int out_stride,
                         float scale, int window, int dims_per_group) {
  extern __shared__ float smem[];
  const int hd = kv.head_dim;
  float* q_s = smem;                       // [hd]
  float* scores = q_s + hd;                // [CHUNK]
  float* part = scores + CHUNK;            // [n_groups][hd]
  __shared__ float red[32];

  const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  TOut* o = out + (size_t)r * out_stride + (size_t)h * hd;
  const int slot = row_slot[r];
  if (slot < 0) {
    for (int i = tid; i < hd; i += THREADS) o[i] = nb_from_f32<TOut>(0.0f);
    return;
  }
  const int pos = row_pos[r];
  const int kvh = h / group;
  const int j_begin = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
  const int j_end = pos + 1;

  const T* qr = q + (size_t)r * q_stride + q_col + (size_t)h * hd;
  for (int i = tid; i < hd; i += THREADS) q_s[i] = nb_to_f32(qr[i]);

  const int n_groups = THREADS / dims_per_group;
  const int dd = tid % dims_per_group, g = tid / dims_per_group;
  float m_run = -INFINITY, l_run = 0.0f, acc = 0.0f;
  __syncthreads();

  for (int c0 = j_begin; c0 < j_end; c0 += CHUNK) {
    const int c1 = min(c0 + CHUNK, j_end);
    // scores of this chunk
    float cmax = -INFINITY;
    for (int j = c0 + tid; j < c1; j += THREADS) {
      const T* kr = kv_row<T>((const T*)kv.k, kv, slot, kvh, j);
      float dot = 0.0f;
      for (int i = 0; i < hd; ++i) dot = fmaf(q_s[i], nb_to_f32(kr[i]), dot);
      const float s = dot * scale;
      scores[j - c0] = s;
      cmax = fmaxf(cmax, s);
    }
    cmax = nb_block_max(cmax, red);
    const float m_new = fmaxf(m_run, cmax);
    float csum = 0.0f;
    for (int j = c0 + tid; j < c1; j += THREADS) {
      const float p = expf(scores[j - c0] - m_new);
      scores[j - c0] = p;
      csum += p;
    }
    csum = nb_block_sum(csum, red);  // also orders the writes of `scores` before the reads below
    const float rescale = (m_run == -INFINITY) ? 0.0f : expf(m_run - m_new);
    l_run = l_run * rescale + csum;
    acc *= rescale;
    if (dd < hd) {
      for (int j = c0 + g; j < c1; j += n_groups) {
        const T* vr = kv_row<T>((const T*)kv.v, kv, slot, kvh, j);
        acc = fmaf(scores[j - c0], nb_to_f32(vr[dd]), acc);
      }
    }
    m_run = m_new;
    __syncthreads();  // `scores` is rewritten by the next chunk
  }

  if (dd < hd) part[g * hd + dd] = acc;
  __syncthreads();
  if (tid < hd) {
    float s = 0.0f;
    for (int gg = 0; gg < n_groups; ++gg) s += part[gg * hd + tid];
    o[tid] = nb_from_f32<TOut>(l_run > 0.0f ? s / l_run : s);
  }
}

template <typename T, typename TOut>
int launch(const void* q, int q_stride, int q_col, const int* row_slot, const int* row_pos,
           const NbPagedKV& kv, int n_heads, void* out, int out_stride, float scale, int window,
           int n_rows, cudaStream_t stream) {
  int dpg = 32;
  while (dpg < kv.head_dim) dpg <<= 1;
  const int n_groups = THREADS / dpg;
  const size_t smem = (size_t)(kv.head_dim + CHUNK + n_groups * kv.head_dim) * sizeof(float);
  dim3 grid(n_rows, n_heads);
  attention_generic_kernel<T, TOut><<<grid, THREADS, smem, stream>>>(
      (const T*)q, q_stride, q_col, row_slot, row_pos, kv, n_heads / kv.n_kv_heads, (TOut*)out,
      out_stride, scale, window, dpg);
  return 0;
}

}  // namespace

// q: packed rows, row r holds head h's query at columns q_col + h*head_dim .. ; same element
// type as the cache.  out: [n_rows][out_stride], head h at columns h*head_dim.
NB_EXPORT int nb_attention_generic(const void* q, int dtype, int q_stride, int q_col,
                                   const int* row_slot, const int* row_pos, const void* k_cache,
                                   const void* v_cache, const int* block_table, int max_pages,
                                   int page, int n_heads, int n_kv_heads, int head_dim, void* out,
                                   int out_dtype, int out_stride, float scale, int window,
                                   int n_rows, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(head_dim >= 1 && head_dim <= 256, NB_ERR_UNSUPPORTED,
             "attention_generic: head size %d is outside 1..256", head_dim);
  NB_REQUIRE(n_kv_heads >= 1 && n_heads % n_kv_heads == 0, NB_ERR_BAD_ARG,
             "attention_generic: %d heads cannot share %d key/value heads", n_heads, n_kv_heads);
  NB_REQUIRE(n_heads <= 65535, NB_ERR_UNSUPPORTED, "attention_generic: too many heads (%d)",
             n_heads);
  NbPagedKV kv{(void*)k_cache, (void*)v_cache, block_table, max_pages, page, n_kv_heads, head_dim};
  typedef __nv_bfloat16 bf16;
  const int key = dtype * 2 + out_dtype;
  switch (key) {
    case 0: launch<float, float>(q, q_stride, q_col, row_slot, row_pos, kv, n_heads, out, out_stride, scale, window, n_rows, stream); break;
    case 1: launch<float, bf16>(q, q_stride, q_col, row_slot, row_pos, kv, n_heads, out, out_stride, scale, window, n_rows, stream); break;
    case 2: launch<bf16, float>(q, q_stride, q_col, row_slot, row_pos, kv, n_heads, out, out_stride, scale, window, n_rows, stream); break;
    case 3: launch<bf16, bf16>(q, q_stride, q_col, row_slot, row_pos, kv, n_heads, out, out_stride, scale, window, n_rows, stream); break;
    default:
      NB_REQUIRE(false, NB_ERR_BAD_ARG, "attention_generic: unknown dtypes %d/%d", dtype, out_dtype);
  }
  NB_CHECK_LAUNCH("attention_generic");
  return 0;
}
