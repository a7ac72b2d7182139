// Prefill attention in true 32-bit arithmetic: many query rows per sequence over the paged
// key/value cache, every product and sum an fp32 multiply-add on the CUDA cores (no tensor
// cores, no rounding of operands).  It is the attention of the whole-model 32-bit path for
// prompts; heads of 64 or 128, pages of 64 tokens.
//
// A CTA takes 64 consecutive query rows of one sequence and one head and walks over the
// sequence's pages up to the last key its rows may see.  Per page: the page's keys (transposed)
// and values go to shared memory; the 16 x 16 threads each compute a 4 x 4 block of the 64 x 64
// scores from the transposed query and key tiles (two 16-byte reads feed 16 multiply-adds);
// scale, causal limit and window; running maximum and sum per row (fp32, maximum subtracted,
// src/ops.rs:6-18) through shuffles among the 16 threads that share a row; probabilities to
// shared memory; then every thread adds its 4 rows x head/16 columns of P V.  Keys after a
// row's own position, before its window or beyond the sequence get no weight, and the rows of
// the last page that hold no key yet are never multiplied with anything.
//
// Reference: src/model.rs:401-422 (scores = dot(q,k)*scale for keys 0..P+i, softmax, weighted
// values); head h reads key/value head h / group (src/model.rs:390).
#include "attention_common.cuh"

namespace {

constexpr int TQ = 64;            // query rows per CTA
constexpr int PAGE_TOKENS = 64;   // keys per page
constexpr int LD = 68;            // floats between rows of a 64-wide shared tile (16-byte aligned)
constexpr int THREADS = 256;

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T, int HD, typename TOut>
__global__ void __launch_bounds__(THREADS)
attention_prefill_f32_kernel(const T* q, int q_stride, int q_col,
                             const int* cu_rows, const int* seq_slot,
                             const int* seq_pos0, NbPagedKV kv, int group,
                             TOut* out, int out_stride, float scale, int window) {
  constexpr int CPT = HD / 16;          // output columns per thread
  constexpr int VLD = HD + 4;           // floats between rows of the value tile
  extern __shared__ __align__(16) float sm[];
  float* Qt = sm;                       // [HD][LD]: Qt[d][i] = q of row i, column d
  float* Kt = Qt + HD * LD;             // [HD][LD]: Kt[d][j] = key j of the page, column d
  float* Vs = Kt + HD * LD;             // [64][VLD]
  float* Ps = Vs + PAGE_TOKENS * VLD;   // [64][LD]: probabilities of the page, row i, key j

  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int tile = blockIdx.x, h = blockIdx.y, s = blockIdx.z;
  const int row0 = cu_rows[s], n_q = cu_rows[s + 1] - row0;
  const int q0 = tile * TQ;
  const int slot = seq_slot[s];
  if (q0 >= n_q || slot < 0) return;
  const int pos0 = seq_pos0[s];
  const int kvh = h / group;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int rows_here = min(TQ, n_q - q0);
  const int last_pos = pos0 + q0 + rows_here - 1;                    // newest key any row sees
  const int first_key = (window > 0) ? max(0, pos0 + q0 + 1 - window) : 0;
  const int p_begin = first_key / PAGE_TOKENS, p_end = last_pos / PAGE_TOKENS + 1;
  const int* table = kv.block_table + (size_t)slot * kv.max_pages;

  // the query tile, transposed; rows beyond the sequence are zero
  for (int idx = tid; idx < TQ * HD; idx += THREADS) {
    const int i = idx / HD, d = idx - i * HD;
    Qt[d * LD + i] = i < rows_here
                         ? to_f32<T>(q[(size_t)(row0 + q0 + i) * q_stride + q_col + (size_t)h * HD + d])
                         : 0.0f;
  }

  float o[4][CPT];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < CPT; ++c) o[i][c] = 0.0f;
  float m_run[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, l_run[4] = {0.0f, 0.0f, 0.0f, 0.0f};

  for (int p = p_begin; p < p_end; ++p) {
    __syncthreads();   // the tiles of the page before are no longer read (and Qt is complete)
    const int page_id = table[p];
    const T* ksrc = (const T*)kv.k + ((size_t)page_id * kv.n_kv_heads + kvh) * PAGE_TOKENS * HD;
    const T* vsrc = (const T*)kv.v + ((size_t)page_id * kv.n_kv_heads + kvh) * PAGE_TOKENS * HD;
    const int keys_here = min(PAGE_TOKENS, last_pos + 1 - p * PAGE_TOKENS);   // rows that hold a key
    for (int idx = tid; idx < PAGE_TOKENS * HD; idx += THREADS) {
      const int j = idx / HD, d = idx - j * HD;
      const bool live = j < keys_here;          // what lies beyond is an earlier owner's: never read
      Kt[d * LD + j] = live ? to_f32<T>(ksrc[idx]) : 0.0f;
      Vs[j * VLD + d] = live ? to_f32<T>(vsrc[idx]) : 0.0f;
    }
    __syncthreads();

    // scores: rows ty*4 + ii, keys tx*4 + jj
    float sc[4][4];
#pragma unroll
    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) sc[ii][jj] = 0.0f;
#pragma unroll 8
    for (int d = 0; d < HD; ++d) {
      const float4 a = *reinterpret_cast<const float4*>(Qt + d * LD + ty * 4);
      const float4 b = *reinterpret_cast<const float4*>(Kt + d * LD + tx * 4);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int ii = 0; ii < 4; ++ii)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) sc[ii][jj] = fmaf(av[ii], bv[jj], sc[ii][jj]);
    }
    // scale, causal limit, window; the row's maximum and sum among the 16 threads of the row
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      const int qp = pos0 + q0 + ty * 4 + ii;          // absolute position of the row's query
      float mx = -INFINITY;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int key = p * PAGE_TOKENS + tx * 4 + jj;
        const bool ok = key <= qp && (window <= 0 || key > qp - window);
        sc[ii][jj] = ok ? sc[ii][jj] * scale : -INFINITY;
        mx = fmaxf(mx, sc[ii][jj]);
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float m_new = fmaxf(m_run[ii], mx);
      const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
      const float resc = (m_run[ii] == -INFINITY) ? 0.0f : expf(m_run[ii] - m_use);
      m_run[ii] = m_new;
      float sum = 0.0f;
      float pr[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        pr[jj] = (sc[ii][jj] == -INFINITY) ? 0.0f : expf(sc[ii][jj] - m_use);
        sum += pr[jj];
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      l_run[ii] = l_run[ii] * resc + sum;
#pragma unroll
      for (int c = 0; c < CPT; ++c) o[ii][c] *= resc;
      *reinterpret_cast<float4*>(Ps + (ty * 4 + ii) * LD + tx * 4) = make_float4(pr[0], pr[1], pr[2], pr[3]);
    }
    __syncthreads();

    // o[ii][c] += sum_j P[row][j] V[j][tx*CPT + c]
#pragma unroll 2
    for (int j = 0; j < PAGE_TOKENS; j += 4) {
      float pv[4][4];
#pragma unroll
      for (int ii = 0; ii < 4; ++ii) {
        const float4 t4 = *reinterpret_cast<const float4*>(Ps + (ty * 4 + ii) * LD + j);
        pv[ii][0] = t4.x; pv[ii][1] = t4.y; pv[ii][2] = t4.z; pv[ii][3] = t4.w;
      }
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        float vv[CPT];
#pragma unroll
        for (int c4 = 0; c4 < CPT / 4; ++c4) {
          const float4 t4 = *reinterpret_cast<const float4*>(Vs + (j + jj) * VLD + tx * CPT + c4 * 4);
          vv[c4 * 4] = t4.x; vv[c4 * 4 + 1] = t4.y; vv[c4 * 4 + 2] = t4.z; vv[c4 * 4 + 3] = t4.w;
        }
#pragma unroll
        for (int ii = 0; ii < 4; ++ii)
#pragma unroll
          for (int c = 0; c < CPT; ++c) o[ii][c] = fmaf(pv[ii][jj], vv[c], o[ii][c]);
      }
    }
  }

#pragma unroll
  for (int ii = 0; ii < 4; ++ii) {
    const int i = ty * 4 + ii;
    if (i >= rows_here) continue;
    const float inv = l_run[ii] > 0.0f ? 1.0f / l_run[ii] : 0.0f;
    TOut* dst = out + (size_t)(row0 + q0 + i) * out_stride + (size_t)h * HD + tx * CPT;
#pragma unroll
    for (int c = 0; c < CPT; ++c) dst[c] = nb_from_f32<TOut>(o[ii][c] * inv);
  }
}

template <typename T, int HD, typename TOut>
int launch(const void* q, int q_stride, int q_col, const int* cu_rows, const int* seq_slot,
           const int* seq_pos0, const NbPagedKV& kv, int n_heads, void* out, int out_stride,
           float scale, int window, int n_seqs, int max_q_len, cudaStream_t stream) {
  const size_t smem = (size_t)(2 * HD * LD + PAGE_TOKENS * (HD + 4) + TQ * LD) * sizeof(float);
  auto kern = attention_prefill_f32_kernel<T, HD, TOut>;
  static bool configured = false;   // per instantiation
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  dim3 grid((max_q_len + TQ - 1) / TQ, n_heads, n_seqs);
  NB_CUDA(nb_launch(kern, grid, dim3(THREADS), smem, stream, (const T*)q, q_stride, q_col, cu_rows,
                    seq_slot, seq_pos0, kv, n_heads / kv.n_kv_heads, (TOut*)out, out_stride, scale,
                    window));
  return 0;
}

}  // namespace

// 1 if the 32-bit prefill kernel takes this shape (otherwise the caller uses the generic kernel).
NB_EXPORT int nb_attention_prefill_f32_supported(int head_dim, int n_heads, int n_kv_heads, int page) {
  if (page != PAGE_TOKENS || n_kv_heads < 1 || n_heads % n_kv_heads != 0) return 0;
  return head_dim == 64 || head_dim == 128;
}

// Rows of sequence s are cu_rows[s]..cu_rows[s+1] of the packed batch, at positions
// seq_pos0[s].. of slot seq_slot[s]; their keys and values are already in the cache.  `dtype`:
// element type of the queries and of the cache (fp32, or bf16 widened on the way in).
NB_EXPORT int nb_attention_prefill_f32(const void* q, int dtype, int q_stride, int q_col,
                                       const int* cu_rows, const int* seq_slot, const int* seq_pos0,
                                       const void* k_cache, const void* v_cache,
                                       const int* block_table, int max_pages, int page, int n_heads,
                                       int n_kv_heads, int head_dim, void* out, int out_dtype,
                                       int out_stride, float scale, int window, int n_seqs,
                                       int max_q_len, cudaStream_t stream) {
  if (n_seqs == 0 || max_q_len == 0) return 0;
  NB_REQUIRE(nb_attention_prefill_f32_supported(head_dim, n_heads, n_kv_heads, page), NB_ERR_UNSUPPORTED,
             "attention_prefill_f32: unsupported shape (head size %d, %d/%d heads, page %d)", head_dim,
             n_heads, n_kv_heads, page);
  NB_REQUIRE(n_seqs <= 65535 && n_heads <= 65535, NB_ERR_UNSUPPORTED, "attention_prefill_f32: grid too large");
  NbPagedKV kv{(void*)k_cache, (void*)v_cache, block_table, max_pages, page, n_kv_heads, head_dim};
  typedef __nv_bfloat16 bf16;
  int rc = NB_ERR_BAD_ARG;
#define NB_ARGS q, q_stride, q_col, cu_rows, seq_slot, seq_pos0, kv, n_heads, out, out_stride, scale, window, n_seqs, max_q_len, stream
#define NB_HD(T_, TO_) rc = head_dim == 64 ? launch<T_, 64, TO_>(NB_ARGS) : launch<T_, 128, TO_>(NB_ARGS)
  if (dtype == NB_F32 && out_dtype == NB_F32) { NB_HD(float, float); }
  else if (dtype == NB_F32 && out_dtype == NB_BF16) { NB_HD(float, bf16); }
  else if (dtype == NB_BF16 && out_dtype == NB_F32) { NB_HD(bf16, float); }
  else if (dtype == NB_BF16 && out_dtype == NB_BF16) { NB_HD(bf16, bf16); }
#undef NB_HD
#undef NB_ARGS
  NB_REQUIRE(rc != NB_ERR_BAD_ARG, NB_ERR_BAD_ARG, "attention_prefill_f32: unknown dtypes %d/%d", dtype, out_dtype);
  if (rc) return rc;
  NB_CHECK_LAUNCH("attention_prefill_f32");
  return 0;
}
