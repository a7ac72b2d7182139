// Decode attention with one CTA per (row, key/value head): sixteen warps, each taking whole
// pages of the sequence (page p belongs to warp p % 16) straight from global memory with
// 16-byte loads, many in flight per lane; the warps' running (max, sum, accumulator) are
// merged through shared memory at the end.  Nothing goes through global scratch and nothing
// waits on another CTA, so a step with few rows and a context of a few dozen pages -- the
// usual decode step of a small model -- costs one trip to memory for the cache plus one
// block-wide merge.  With few (row, head) pairs and a very long context the split kernel
// (attention_decode.cu) spreads one pair over several CTAs instead; the caller chooses.
//
// Arithmetic is the same as there: scores = dot(q, k) * scale over keys 0..pos (or the last
// `window`), softmax and weighted values in fp32 (src/model.rs:401-422); query head h reads
// key/value head h / group (src/model.rs:390).  With `append` the row's own key and value
// (columns k_col / v_col of the same buffer) are written to the cache and attended to.
#include "attention_common.cuh"

namespace {

constexpr int PAGE_TOKENS = 64;

// NW warps per CTA: sixteen, or eight when many query heads share the key/value head (their
// accumulators need the registers).
template <typename T, int HD, int G, int NW, typename TOut>
__global__ void __launch_bounds__(NW * 32)
attention_decode_wide_kernel(const T* __restrict__ q, int q_stride, int q_col,
                             const int* __restrict__ row_slot, const int* __restrict__ row_pos,
                             NbPagedKV kv, int group, TOut* __restrict__ out, int out_stride,
                             float scale, int window, int append, int k_col, int v_col) {
  constexpr int EPL = Lane16<T>::N;           // elements per lane
  constexpr int LPR = HD / EPL;               // lanes per key row
  constexpr int RPW = 32 / LPR;               // key rows per warp step
  constexpr int STEPS = PAGE_TOKENS / RPW;    // steps per page
  constexpr int UNR = STEPS < 8 ? STEPS : 8;  // steps whose loads are in flight together
  static_assert(LPR >= 1 && LPR <= 32 && (LPR & (LPR - 1)) == 0, "head size not supported");

  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* w_acc = reinterpret_cast<float*>(smem_raw);      // [WARPS][G][HD]
  float* w_ml = w_acc + NW * G * HD;               // [WARPS][G][2]

  nb_launch_dependents();
  nb_grid_dependency_wait();
  const int kvh = blockIdx.x, r = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sub = lane / LPR, part = lane % LPR;
  const int slot = row_slot[r];
  if (slot < 0) {   // padding row
    for (int i = tid; i < group * HD; i += (NW * 32))
      out[(size_t)r * out_stride + (size_t)kvh * group * HD + i] = nb_from_f32<TOut>(0.0f);
    return;
  }
  const int pos = row_pos[r];
  const int kv_len = pos + 1;
  const int j_begin = (window > 0 && kv_len > window) ? kv_len - window : 0;
  const int first_page = j_begin / PAGE_TOKENS;
  const int end_page = (kv_len + PAGE_TOKENS - 1) / PAGE_TOKENS;
  const int* table = kv.block_table + (size_t)slot * kv.max_pages;
  const T* qrow = q + (size_t)r * q_stride;

  float qreg[G][EPL];
#pragma unroll
  for (int gh = 0; gh < G; ++gh) {
    if (gh < group) {
      Lane16<T>::load(qrow + q_col + (size_t)(kvh * group + gh) * HD + part * EPL, qreg[gh]);
    } else {
#pragma unroll
      for (int e = 0; e < EPL; ++e) qreg[gh][e] = 0.0f;
    }
  }
  float m_run[G], l_run[G], acc[G][EPL];
#pragma unroll
  for (int gh = 0; gh < G; ++gh) {
    m_run[gh] = -INFINITY;
    l_run[gh] = 0.0f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[gh][e] = 0.0f;
  }

  for (int p = first_page + warp; p < end_page; p += NW) {
    const int page_id = table[p];
    const size_t page_off = ((size_t)page_id * kv.n_kv_heads + kvh) * PAGE_TOKENS * HD;
    T* kpage = (T*)kv.k + page_off;
    T* vpage = (T*)kv.v + page_off;
#pragma unroll 1
    for (int s0 = 0; s0 < STEPS; s0 += UNR) {
      if (p * PAGE_TOKENS + s0 * RPW >= kv_len) break;   // the rest of the page is unused
      uint4 kraw[UNR], vraw[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int row = (s0 + u) * RPW + sub;
        const int j = p * PAGE_TOKENS + row;
        const bool own = append && j == pos;   // this step's own token: not in the cache yet
        const T* kp = own ? qrow + k_col + (size_t)kvh * HD + part * EPL
                          : kpage + row * HD + part * EPL;
        const T* vp = own ? qrow + v_col + (size_t)kvh * HD + part * EPL
                          : vpage + row * HD + part * EPL;
        if (j < kv_len) {
          kraw[u] = *reinterpret_cast<const uint4*>(kp);
          vraw[u] = *reinterpret_cast<const uint4*>(vp);
          if (own) {
            *reinterpret_cast<uint4*>(kpage + row * HD + part * EPL) = kraw[u];
            *reinterpret_cast<uint4*>(vpage + row * HD + part * EPL) = vraw[u];
          }
        } else {
          kraw[u] = make_uint4(0u, 0u, 0u, 0u);
          vraw[u] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int j = p * PAGE_TOKENS + (s0 + u) * RPW + sub;
        const bool valid = (j >= j_begin) && (j < kv_len);
        float kf[EPL], vf[EPL];
        Lane16<T>::unpack(kraw[u], kf);
        Lane16<T>::unpack(vraw[u], vf);
#pragma unroll
        for (int gh = 0; gh < G; ++gh) {
          float dot = 0.0f;
#pragma unroll
          for (int e = 0; e < EPL; ++e) dot = fmaf(qreg[gh][e], kf[e], dot);
#pragma unroll
          for (int o = LPR / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
          const float s = valid ? dot * scale : -INFINITY;
          float mx = s;
#pragma unroll
          for (int o = LPR; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
          const float m_new = fmaxf(m_run[gh], mx);
          if (m_new > -INFINITY) {   // warp-uniform
            const float rescale = (m_run[gh] == -INFINITY) ? 0.0f : expf(m_run[gh] - m_new);
            const float pr = valid ? expf(s - m_new) : 0.0f;
            l_run[gh] = l_run[gh] * rescale + pr;
#pragma unroll
            for (int e = 0; e < EPL; ++e) acc[gh][e] = fmaf(pr, vf[e], acc[gh][e] * rescale);
            m_run[gh] = m_new;
          }
        }
      }
    }
  }

  // key rows a warp handled side by side (lanes with equal `part`), then the warps
#pragma unroll
  for (int gh = 0; gh < G; ++gh) {
#pragma unroll
    for (int o = LPR; o < 32; o <<= 1) {
      l_run[gh] += __shfl_xor_sync(0xffffffffu, l_run[gh], o);
#pragma unroll
      for (int e = 0; e < EPL; ++e) acc[gh][e] += __shfl_xor_sync(0xffffffffu, acc[gh][e], o);
    }
    if (sub == 0) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) w_acc[(warp * G + gh) * HD + part * EPL + e] = acc[gh][e];
      if (part == 0) {
        w_ml[(warp * G + gh) * 2] = m_run[gh];
        w_ml[(warp * G + gh) * 2 + 1] = l_run[gh];
      }
    }
  }
  __syncthreads();
  for (int i = tid; i < group * HD; i += (NW * 32)) {
    const int gh = i / HD, c = i - gh * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, w_ml[(w * G + gh) * 2]);
    float a = 0.0f, l = 0.0f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float mw = w_ml[(w * G + gh) * 2];
      const float f = (mw == -INFINITY) ? 0.0f : expf(mw - M);
      a += f * w_acc[(w * G + gh) * HD + c];
      l += f * w_ml[(w * G + gh) * 2 + 1];
    }
    out[(size_t)r * out_stride + (size_t)(kvh * group + gh) * HD + c] =
        nb_from_f32<TOut>(l > 0.0f ? a / l : a);
  }
}

template <typename T, int HD, int G, typename TOut>
int launch(const void* q, int q_stride, int q_col, const int* row_slot, const int* row_pos,
           const NbPagedKV& kv, int group, void* out, int out_stride, float scale, int window,
           int n_rows, int append, int k_col, int v_col, cudaStream_t stream) {
  constexpr int NW = G <= 2 ? 16 : 8;
  const size_t smem = (size_t)(NW * G * HD + NW * G * 2) * sizeof(float);
  auto kern = attention_decode_wide_kernel<T, HD, G, NW, TOut>;
  if (smem > 48 * 1024)
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  NB_CUDA(nb_launch(kern, dim3(kv.n_kv_heads, n_rows), dim3((NW * 32)), smem, stream, (const T*)q,
                    q_stride, q_col, row_slot, row_pos, kv, group, (TOut*)out, out_stride, scale,
                    window, append, k_col, v_col));
  return 0;
}

template <typename T, int HD, typename TOut>
int by_group(int group, const void* q, int q_stride, int q_col, const int* row_slot,
             const int* row_pos, const NbPagedKV& kv, void* out, int out_stride, float scale,
             int window, int n_rows, int ap, int kc, int vc, cudaStream_t st) {
#define NB_G(G_) \
  return launch<T, HD, G_, TOut>(q, q_stride, q_col, row_slot, row_pos, kv, group, out, out_stride, scale, window, n_rows, ap, kc, vc, st)
  if (group == 1) NB_G(1);
  if (group == 2) NB_G(2);
  if (group <= 4) NB_G(4);
  NB_G(8);
#undef NB_G
}

template <typename T, typename TOut>
int by_head_dim(int hd, int group, const void* q, int q_stride, int q_col, const int* row_slot,
                const int* row_pos, const NbPagedKV& kv, void* out, int out_stride, float scale,
                int window, int n_rows, int ap, int kc, int vc, cudaStream_t st) {
#define NB_HD(HD_) \
  return by_group<T, HD_, TOut>(group, q, q_stride, q_col, row_slot, row_pos, kv, out, out_stride, scale, window, n_rows, ap, kc, vc, st)
  switch (hd) {
    case 16: NB_HD(16);
    case 32: NB_HD(32);
    case 64: NB_HD(64);
    case 128: NB_HD(128);
  }
#undef NB_HD
  return NB_ERR_UNSUPPORTED;
}

}  // namespace

// Same shapes as nb_attention_decode (see nb_attention_decode_supported); no scratch.  The
// rows of `q` must be 16-byte aligned, as must k_col / v_col when `append` is set.
NB_EXPORT int nb_attention_decode_wide(const void* q, int dtype, int q_stride, int q_col,
                                       const int* row_slot, const int* row_pos,
                                       const void* k_cache, const void* v_cache,
                                       const int* block_table, int max_pages, int page,
                                       int n_heads, int n_kv_heads, int head_dim, void* out,
                                       int out_dtype, int out_stride, float scale, int window,
                                       int n_rows, int append, int k_col, int v_col,
                                       cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(page == PAGE_TOKENS && n_kv_heads >= 1 && n_heads % n_kv_heads == 0 &&
                 n_heads / n_kv_heads <= 8 &&
                 (head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128) &&
                 (dtype == NB_F32 || dtype == NB_BF16),
             NB_ERR_UNSUPPORTED,
             "attention_decode_wide: unsupported shape (head size %d, %d/%d heads, page %d)",
             head_dim, n_heads, n_kv_heads, page);
  NB_REQUIRE(n_rows <= 65535, NB_ERR_UNSUPPORTED, "attention_decode_wide: too many rows");
  const int epl = dtype == NB_F32 ? 4 : 8;
  NB_REQUIRE(q_stride % epl == 0 && q_col % epl == 0 && (uintptr_t)q % 16 == 0 &&
                 (!append || (k_col % epl == 0 && v_col % epl == 0)),
             NB_ERR_UNSUPPORTED, "attention_decode_wide: rows must be 16-byte aligned");
  NbPagedKV kv{(void*)k_cache, (void*)v_cache, block_table, max_pages, page, n_kv_heads, head_dim};
  const int group = n_heads / n_kv_heads;
  typedef __nv_bfloat16 bf16;
  int rc;
#define NB_ARGS head_dim, group, q, q_stride, q_col, row_slot, row_pos, kv, out, out_stride, scale, window, n_rows, append, k_col, v_col, stream
  if (dtype == NB_F32)
    rc = out_dtype == NB_F32 ? by_head_dim<float, float>(NB_ARGS) : by_head_dim<float, bf16>(NB_ARGS);
  else
    rc = out_dtype == NB_F32 ? by_head_dim<bf16, float>(NB_ARGS) : by_head_dim<bf16, bf16>(NB_ARGS);
#undef NB_ARGS
  if (rc) return rc;
  NB_CHECK_LAUNCH("attention_decode_wide");
  return 0;
}
