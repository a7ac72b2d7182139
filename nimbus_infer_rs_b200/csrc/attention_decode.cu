// Decode attention: one query row per sequence over that sequence's paged keys and values.
//
// The work is reading the cache once, so the kernel is laid out for bandwidth: a CTA takes one
// (row, key/value head, split of the sequence's pages), streams whole pages (64 keys x head_dim,
// contiguous) into shared memory with 16-byte cp.async copies, two or four pages in flight (the
// first ones asked for before the kernel's wait on its predecessor), and all query heads that
// share the key/value head are served from the same staged page.  Scores, softmax and the
// weighted sum are fp32; every warp keeps a running (max, sum, accumulator) for its quarter of
// a page (the bfloat16 kernel has four warps on a page, or eight on two pages at a time), the
// warps are merged at the end of the split, and the splits are merged either inside a
// thread-block cluster (2 to 8 splits of the bfloat16 kernel: partial results into the first
// CTA's shared memory, one cluster barrier) or by whichever CTA of the (row, head) finishes
// last (a counter in scratch memory that it leaves at zero again).
//
// Scratch (caller-allocated): part_acc [rows][heads][splits][head_dim] fp32, part_ml
// [rows][heads][splits][2] fp32, counters [rows][kv_heads] int32, zero before the first use.
//
// Reference: src/model.rs:401-422 (scores = dot(q,k)*scale over keys 0..pos, softmax,
// weighted values), head h reads key/value head h / group (src/model.rs:390).
#include <mutex>

#include "common.cuh"
#include <atomic>

#include "attention_common.cuh"

namespace {

constexpr int THREADS = 128;
constexpr int WARPS = 4;
constexpr int PAGE_TOKENS = 64;
constexpr int MAX_CLUSTER = 8;   // most splits that one thread-block cluster merges (portable size)

// G: query heads per key/value head served by one CTA (group <= G).
template <typename T, int HD, int G, typename TOut>
__global__ void __launch_bounds__(THREADS)
attention_decode_kernel(const T* q, int q_stride, int q_col,
                        const int* row_slot, const int* row_pos,
                        NbPagedKV kv, int group, TOut* out, int out_stride,
                        float scale, int window, int n_splits, float* part_acc,
                        float* part_ml, int* counters, int append,
                        int k_col, int v_col) {
  constexpr int EPL = Lane16<T>::N;           // elements per lane
  constexpr int LPR = HD / EPL;               // lanes per key row
  constexpr int RPW = 32 / LPR;               // key rows per warp iteration
  constexpr int KEYS_PER_WARP = PAGE_TOKENS / WARPS;
  constexpr int ITERS = KEYS_PER_WARP / RPW;
  constexpr int TILE = PAGE_TOKENS * HD;      // elements of one page of one head
  static_assert(LPR >= 1 && LPR <= 32 && (LPR & (LPR - 1)) == 0, "head size not supported");
  static_assert(ITERS >= 1, "head size not supported");

  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* tiles = reinterpret_cast<T*>(smem_raw);                       // [2 stages][K tile | V tile]
  float* q_s = reinterpret_cast<float*>(smem_raw + (size_t)4 * TILE * sizeof(T));  // [G][HD]
  float* w_acc = q_s + G * HD;                                     // [WARPS][G][HD]
  float* w_ml = w_acc + WARPS * G * HD;                            // [WARPS][G][2]
  __shared__ int s_last;

  nb_grid_dependency_wait();
  const int split = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sub = lane / LPR, part = lane % LPR;
  const int n_heads = kv.n_kv_heads * group;
  const int slot = row_slot[r];
  if (slot < 0) {   // padding row: zeros, written by split 0
    if (split == 0)
      for (int i = tid; i < group * HD; i += THREADS)
        out[(size_t)r * out_stride + (size_t)kvh * group * HD + i] = nb_from_f32<TOut>(0.0f);
    return;
  }
  const int pos = row_pos[r];
  const int kv_len = pos + 1;
  const int j_begin = (window > 0 && kv_len > window) ? kv_len - window : 0;
  const int first_page = j_begin / PAGE_TOKENS;
  const int n_pages = (kv_len + PAGE_TOKENS - 1) / PAGE_TOKENS - first_page;
  const int per_split = (n_pages + n_splits - 1) / n_splits;
  const int p_begin = first_page + split * per_split;
  const int p_end = min(first_page + n_pages, p_begin + per_split);

  // queries of the group, fp32
  for (int i = tid; i < G * HD; i += THREADS) {
    const int gh = i / HD, c = i - gh * HD;
    q_s[i] = (gh < group)
                 ? nb_to_f32(q[(size_t)r * q_stride + q_col + (size_t)(kvh * group + gh) * HD + c])
                 : 0.0f;
  }

  const int* table = kv.block_table + (size_t)slot * kv.max_pages;
  auto issue = [&](int page_idx, int stage) {
    const int page_id = table[page_idx];
    const T* ksrc = (const T*)kv.k + ((size_t)page_id * kv.n_kv_heads + kvh) * TILE;
    const T* vsrc = (const T*)kv.v + ((size_t)page_id * kv.n_kv_heads + kvh) * TILE;
    T* kdst = tiles + (size_t)stage * 2 * TILE;
    T* vdst = kdst + TILE;
    constexpr int VECS = TILE / EPL;   // 16-byte pieces per tile
    for (int i = tid; i < VECS; i += THREADS) {
      cp_async16(kdst + i * EPL, ksrc + i * EPL);
      cp_async16(vdst + i * EPL, vsrc + i * EPL);
    }
    cp_async_commit();
  };

  float m_run[G], l_run[G], acc[G][EPL];
#pragma unroll
  for (int gh = 0; gh < G; ++gh) {
    m_run[gh] = -INFINITY;
    l_run[gh] = 0.0f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[gh][e] = 0.0f;
  }

  if (p_begin < p_end) issue(p_begin, 0);
  __syncthreads();   // q_s is complete
  float qreg[G][EPL];
#pragma unroll
  for (int gh = 0; gh < G; ++gh)
#pragma unroll
    for (int e = 0; e < EPL; ++e) qreg[gh][e] = q_s[gh * HD + part * EPL + e];

  for (int p = p_begin; p < p_end; ++p) {
    const int stage = (p - p_begin) & 1;
    if (p + 1 < p_end) {
      issue(p + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    T* kt = tiles + (size_t)stage * 2 * TILE;
    T* vt = kt + TILE;
    if (append && p == pos / PAGE_TOKENS) {
      // this step's own key and value (row r of the projection output) belong at token `pos`
      // of this page: put them into the staged tile and into the cache
      const int in_page = pos % PAGE_TOKENS;
      const int page_id = table[p];
      for (int i = tid; i < 2 * LPR; i += THREADS) {
        const bool is_v = i >= LPR;
        const int c = (is_v ? i - LPR : i) * EPL;
        const uint4 val = *reinterpret_cast<const uint4*>(
            q + (size_t)r * q_stride + (is_v ? v_col : k_col) + (size_t)kvh * HD + c);
        *reinterpret_cast<uint4*>((is_v ? vt : kt) + in_page * HD + c) = val;
        T* cache = (T*)(is_v ? kv.v : kv.k);
        *reinterpret_cast<uint4*>(cache + ((size_t)page_id * kv.n_kv_heads + kvh) * TILE +
                                  in_page * HD + c) = val;
      }
      __syncthreads();
    }
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int row = warp * KEYS_PER_WARP + it * RPW + sub;   // key within the page
      const int j = p * PAGE_TOKENS + row;
      const bool valid = (j >= j_begin) && (j < kv_len);
      float kf[EPL], vf[EPL];
      Lane16<T>::load(kt + (size_t)row * HD + part * EPL, kf);
      Lane16<T>::load(vt + (size_t)row * HD + part * EPL, vf);
      if (!valid) {   // whatever an unused cache row holds must not reach the sum
#pragma unroll
        for (int e = 0; e < EPL; ++e) vf[e] = 0.0f;
      }
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
    __syncthreads();   // the stage is free for the copy after next
  }

  nb_launch_dependents();   // the pages are read: the next kernel may be set up
  // merge the key rows a warp handled side by side (lanes with equal `part`)
#pragma unroll
  for (int gh = 0; gh < G; ++gh) {
    // l_run of a lane counts only its own rows; every lane of a row group holds the same value
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
  // merge the warps -> partial result of this split
  for (int i = tid; i < group * HD; i += THREADS) {
    const int gh = i / HD, c = i - gh * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, w_ml[(w * G + gh) * 2]);
    float a = 0.0f, l = 0.0f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float mw = w_ml[(w * G + gh) * 2];
      const float f = (mw == -INFINITY) ? 0.0f : expf(mw - M);
      a += f * w_acc[(w * G + gh) * HD + c];
      l += f * w_ml[(w * G + gh) * 2 + 1];
    }
    const int head = kvh * group + gh;
    if (n_splits == 1) {   // nothing to merge with: this is the result
      out[(size_t)r * out_stride + (size_t)head * HD + c] = nb_from_f32<TOut>(l > 0.0f ? a / l : a);
      continue;
    }
    const size_t pi = ((size_t)r * n_heads + head) * n_splits + split;
    part_acc[pi * HD + c] = a;
    if (c == 0) {
      part_ml[pi * 2] = M;
      part_ml[pi * 2 + 1] = l;
    }
  }
  if (n_splits == 1) return;
  // the CTA that finishes last for this (row, key/value head) merges the splits
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&counters[r * kv.n_kv_heads + kvh], 1);
    s_last = (old == n_splits - 1);
    if (s_last) counters[r * kv.n_kv_heads + kvh] = 0;   // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int i = tid; i < group * HD; i += THREADS) {
    const int gh = i / HD, c = i - gh * HD;
    const int head = kvh * group + gh;
    const size_t base = ((size_t)r * n_heads + head) * n_splits;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, __ldcg(&part_ml[(base + s) * 2]));
    float a = 0.0f, l = 0.0f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = __ldcg(&part_ml[(base + s) * 2]);
      const float f = (ms == -INFINITY) ? 0.0f : expf(ms - M);
      a += f * __ldcg(&part_acc[(base + s) * HD + c]);
      l += f * __ldcg(&part_ml[(base + s) * 2 + 1]);
    }
    out[(size_t)r * out_stride + (size_t)head * HD + c] = nb_from_f32<TOut>(l > 0.0f ? a / l : a);
  }
}

// ---------------------------------------------------------------------------------------
// The same job on the tensor cores, for a bf16 cache.  The CUDA-core kernel above spends its
// time on instructions (widening every key and value, shuffles, a running softmax per four
// keys); here a warp's 16 keys of a page are one mma.sync operand: scores = K (16 keys x
// head_dim) times Q^T (head_dim x 8 query heads of the group, unused columns zero), then the
// value product out^T (head_dim x 8 heads) += V^T (head_dim x 16 keys) times P (16 keys x 8
// heads).  Softmax statistics stay fp32 per head (in units of log2 e); probabilities are
// rounded to bf16 only as the operand of the value product, as in the prefill kernel.  Pages
// are staged with padded rows so that ldmatrix runs without bank conflicts.  Any head size
// that is a multiple of 16 up to 128; up to 8 query heads per key/value head at no extra cost.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// MMA_STAGES: pages (keys and values) in flight per CTA; NW: warps.  Four warps share a page
// (16 keys each).  A page costs a warp about 1,400 clocks of dependent steps (loads from
// shared memory, two rounds of tensor-core instructions with the softmax between them), so
// when the CTAs of a launch fit on the GPU with four pages each, eight warps take two pages
// at a time; a large batch has four warps and two pages per CTA, for more CTAs per SM.
template <int HD, typename TOut, int MMA_STAGES, bool CLUSTERED, int NW>
__global__ void __launch_bounds__(NW * 32)
attention_decode_mma_kernel(const __nv_bfloat16* q, int q_stride, int q_col,
                            const int* row_slot, const int* row_pos,
                            NbPagedKV kv, int group, TOut* out, int out_stride,
                            float scale, int window, int n_splits, float* part_acc,
                            float* part_ml, int* counters, int append,
                            int k_col, int v_col) {
  typedef __nv_bfloat16 bf16;
  constexpr bool clustered = CLUSTERED;
  constexpr int ROW = HD + 8;          // padded row of a staged page (elements)
  constexpr int KS = HD / 16;          // k-steps of the score product = row tiles of the value product
  constexpr int GH = 8;                // query heads an MMA column block holds
  constexpr int NT = NW * 32;          // threads
  constexpr int PPI = NW / 4;          // pages per turn of the loop
  static_assert((NW == 4 || NW == 8) && MMA_STAGES % PPI == 0, "four or eight warps");
  constexpr int TILE = PAGE_TOKENS * HD;
  constexpr int STILE = PAGE_TOKENS * ROW;
  static_assert(HD % 16 == 0 && HD >= 16 && HD <= 128, "head size not supported");

  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* tiles = reinterpret_cast<bf16*>(smem_raw);                   // [stages][K | V][64][ROW]
  // the warps' partial results, after the last page has been read: over the page tiles
  // (more CTAs fit on an SM that way)
  float* w_acc = reinterpret_cast<float*>(smem_raw);                 // [NW][GH][HD]
  float* w_ml = w_acc + NW * GH * HD;                                // [NW][GH][2]
  static_assert((size_t)(NW * GH * HD + NW * GH * 2) * sizeof(float) <=
                    (size_t)2 * MMA_STAGES * STILE * sizeof(bf16), "partial results must fit in the page tiles");
  __shared__ int s_last;
  // clustered: the splits of a row and key-value head are one thread-block cluster (split =
  // rank); they hand their partial results to split 0 through its shared memory, in a region
  // of its own behind the page tiles, instead of through global memory and a counter
  float* c_part = reinterpret_cast<float*>(smem_raw + (size_t)2 * MMA_STAGES * STILE * sizeof(bf16));

  // Before the wait: where the row's pages lie, and its first pages on their way.  The batch
  // layout, the block table and the pages were written at least two kernels ago (earlier
  // steps, host copies); the only thing the kernel in front of this one writes is the step's
  // own rows (queries, and the new key and value, which are patched into the staged page
  // after the wait).
  const int split = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int wq = warp & 3, po = warp >> 2;   // quarter of a page, page of a turn
  const int n_heads = kv.n_kv_heads * group;
  const int slot = row_slot[r];
  if (slot < 0) {   // padding row: zeros, written by split 0
    nb_grid_dependency_wait();
    nb_launch_dependents();
    if (split == 0)
      for (int i = tid; i < group * HD; i += NT)
        out[(size_t)r * out_stride + (size_t)kvh * group * HD + i] = nb_from_f32<TOut>(0.0f);
    return;
  }
  const int pos = row_pos[r];
  const int kv_len = pos + 1;
  const int j_begin = (window > 0 && kv_len > window) ? kv_len - window : 0;
  const int first_page = j_begin / PAGE_TOKENS;
  const int n_pages = (kv_len + PAGE_TOKENS - 1) / PAGE_TOKENS - first_page;
  const int per_split = (n_pages + n_splits - 1) / n_splits;
  const int p_begin = first_page + split * per_split;
  const int p_end = min(first_page + n_pages, p_begin + per_split);
  const int* table = kv.block_table + (size_t)slot * kv.max_pages;
  const bf16* qrow = q + (size_t)r * q_stride;

  auto issue = [&](int page_idx, int stage) {
    const int page_id = table[page_idx];
    const bf16* ksrc = (const bf16*)kv.k + ((size_t)page_id * kv.n_kv_heads + kvh) * TILE;
    const bf16* vsrc = (const bf16*)kv.v + ((size_t)page_id * kv.n_kv_heads + kvh) * TILE;
    bf16* kdst = tiles + (size_t)stage * 2 * STILE;
    bf16* vdst = kdst + STILE;
    constexpr int CPR = HD / 8;   // 16-byte pieces per row
    for (int i = tid; i < PAGE_TOKENS * CPR; i += NT) {
      const int row = i / CPR, c = i - row * CPR;
      cp_async16(kdst + row * ROW + c * 8, ksrc + row * HD + c * 8);
      cp_async16(vdst + row * ROW + c * 8, vsrc + row * HD + c * 8);
    }
  };
  // one commit group per stage of the ring, also an empty one: the count of groups in flight
  // then says which page has landed
#pragma unroll
  for (int i = 0; i < MMA_STAGES; ++i) {
    if (p_begin + i < p_end) issue(p_begin + i, i);
    cp_async_commit();
  }

  nb_grid_dependency_wait();
  // Every CTA of a cluster says that it runs (a padding row's CTAs have all left above); the
  // matching wait stands in front of the first store into another CTA's shared memory.
  if constexpr (clustered) asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory");

  // Q^T as the B operand of the score product: column g of the block is query head g of the
  // group (zero beyond the group); this thread holds rows 2t, 2t+1 and 2t+8, 2t+9 of each k-step
  uint32_t qb[KS][2];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    qb[ks][0] = qb[ks][1] = 0u;
    if (g < group) {
      const bf16* p = qrow + q_col + (size_t)(kvh * group + g) * HD + ks * 16 + 2 * t;
      qb[ks][0] = *reinterpret_cast<const uint32_t*>(p);
      qb[ks][1] = *reinterpret_cast<const uint32_t*>(p + 8);
    }
  }

  // this thread's share: heads 2t and 2t+1; keys g and g+8 of the warp's 16; rows g, g+8 of
  // every 16-row tile of the output
  float o[KS][4];
#pragma unroll
  for (int i = 0; i < KS; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  const float sl2 = scale * 1.4426950408889634f;

  int stage = 0;
  for (int p0 = p_begin; p0 < p_end; p0 += PPI) {
    cp_async_wait<MMA_STAGES - PPI>();   // all but the newest groups: the turn's pages are in
    __syncthreads();
#pragma unroll
    for (int q2 = 0; q2 < PPI; ++q2) {
    const int p = p0 + q2;
    if (p >= p_end) break;
    bf16* kt = tiles + (size_t)(stage + q2) * 2 * STILE;
    bf16* vt = kt + STILE;
    const bool own_page = append && p == pos / PAGE_TOKENS;
    const int tail_row = kv_len - p * PAGE_TOKENS;   // first row of the page that holds no key yet
    if (own_page || tail_row < PAGE_TOKENS) {        // uniform over the CTA
      constexpr int CPR = HD / 8;
      if (own_page) {
        // this step's own key and value belong at token `pos` of this page: into the staged
        // tile and into the cache
        const int in_page = pos % PAGE_TOKENS;
        const int page_id = table[p];
        for (int i = tid; i < 2 * CPR; i += NT) {
          const bool is_v = i >= CPR;
          const int c = (is_v ? i - CPR : i) * 8;
          const uint4 val = *reinterpret_cast<const uint4*>(
              qrow + (is_v ? v_col : k_col) + (size_t)kvh * HD + c);
          *reinterpret_cast<uint4*>((is_v ? vt : kt) + in_page * ROW + c) = val;
          bf16* cache = (bf16*)(is_v ? kv.v : kv.k);
          *reinterpret_cast<uint4*>(cache + ((size_t)page_id * kv.n_kv_heads + kvh) * TILE +
                                    in_page * HD + c) = val;
        }
      }
      // Rows of the page after the sequence's last key hold whatever an earlier owner of the
      // page left there.  Their probabilities are zero, but zero times a non-finite value is
      // not: the value rows are cleared in the staged copy (a masked score needs no such care,
      // it is replaced, not multiplied).
      for (int i = tid; i < (PAGE_TOKENS - tail_row) * CPR; i += NT) {
        const int row = tail_row + i / CPR, c = (i % CPR) * 8;
        *reinterpret_cast<uint4*>(vt + row * ROW + c) = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncthreads();
    }
    }
    const int p = p0 + po;                            // this warp's page
    bf16* kt = tiles + (size_t)(stage + po) * 2 * STILE;
    bf16* vt = kt + STILE;
    const int key0 = p * PAGE_TOKENS + wq * 16;       // first key of this warp's 16
    if (p < p_end && key0 < kv_len && key0 + 16 > j_begin) {   // warp-uniform: something to attend to
      // the k-steps of the score product in accumulators of their own, added up afterwards:
      // a tensor-core instruction takes long to hand its result to the next one
      float sck[KS < 4 ? KS : 4][4];
#pragma unroll
      for (int i = 0; i < (KS < 4 ? KS : 4); ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) sck[i][j] = 0.0f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t ka[4];
        ldsm_x4(ka, kt + (wq * 16 + (lane & 15)) * ROW + ks * 16 + (lane >> 4) * 8);
        mma_16816(sck[ks & 3], ka, qb[ks][0], qb[ks][1]);
      }
      float sc[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a = sck[0][j];
#pragma unroll
        for (int i = 1; i < (KS < 4 ? KS : 4); ++i) a += sck[i][j];
        sc[j] = a;
      }
      const int ja = key0 + g, jb = ja + 8;
      const bool va = ja >= j_begin && ja < kv_len, vb = jb >= j_begin && jb < kv_len;
      const float s0 = va ? sc[0] * sl2 : -INFINITY, s1 = va ? sc[1] * sl2 : -INFINITY;
      const float s2 = vb ? sc[2] * sl2 : -INFINITY, s3 = vb ? sc[3] * sl2 : -INFINITY;
      float mx0 = fmaxf(s0, s2), mx1 = fmaxf(s1, s3);
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
      }
      const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);   // finite: a key is valid
      const float r0 = (m_run[0] == -INFINITY) ? 0.0f : nb_exp2(m_run[0] - mn0);
      const float r1 = (m_run[1] == -INFINITY) ? 0.0f : nb_exp2(m_run[1] - mn1);
      m_run[0] = mn0;
      m_run[1] = mn1;
      const float p0 = nb_exp2(s0 - mn0), p1 = nb_exp2(s1 - mn1);
      const float p2 = nb_exp2(s2 - mn0), p3 = nb_exp2(s3 - mn1);
      l_run[0] = l_run[0] * r0 + p0 + p2;
      l_run[1] = l_run[1] * r1 + p1 + p3;
#pragma unroll
      for (int i = 0; i < KS; ++i) {
        o[i][0] *= r0; o[i][1] *= r1; o[i][2] *= r0; o[i][3] *= r1;
      }
      // P as the B operand of the value product: this thread needs keys 2t, 2t+1 (and +8) of
      // head g; they sit in lanes (g' = 2t, t' = g/2) and (g' = 2t+1, t' = g/2)
      const uint32_t pe = pack2_bf16(p0, p2);   // head 2t:   keys g, g+8
      const uint32_t po = pack2_bf16(p1, p3);   // head 2t+1: keys g, g+8
      const int src1 = (2 * t) * 4 + (g >> 1), src2 = src1 + 4;
      const uint32_t e1 = __shfl_sync(0xffffffffu, pe, src1), o1 = __shfl_sync(0xffffffffu, po, src1);
      const uint32_t e2 = __shfl_sync(0xffffffffu, pe, src2), o2 = __shfl_sync(0xffffffffu, po, src2);
      const uint32_t x1 = (g & 1) ? o1 : e1, x2 = (g & 1) ? o2 : e2;
      const uint32_t pb0 = __byte_perm(x1, x2, 0x5410);   // keys 2t, 2t+1
      const uint32_t pb1 = __byte_perm(x1, x2, 0x7632);   // keys 2t+8, 2t+9
#pragma unroll
      for (int i = 0; i < KS; ++i) {
        uint32_t va4[4];
        ldsm_x4_trans(va4, vt + (wq * 16 + (lane & 7) + (lane >> 4) * 8) * ROW + i * 16 +
                               ((lane >> 3) & 1) * 8);
        mma_16816(o[i], va4, pb0, pb1);
      }
    }
    __syncthreads();   // the stages are free: the pages after the ones in flight go there
#pragma unroll
    for (int q2 = 0; q2 < PPI; ++q2) {
      if (p0 + q2 + MMA_STAGES < p_end) issue(p0 + q2 + MMA_STAGES, stage + q2);
      cp_async_commit();
    }
    stage += PPI;
    if (stage == MMA_STAGES) stage = 0;
  }
  cp_async_wait<0>();

  nb_launch_dependents();   // the pages are read: the next kernel may be set up
  // row sums over the lanes that share a head (different keys), then the warps
#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], off);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], off);
  }
#pragma unroll
  for (int i = 0; i < KS; ++i) {
    float* base = w_acc + (size_t)warp * GH * HD;
    base[(2 * t) * HD + i * 16 + g] = o[i][0];
    base[(2 * t + 1) * HD + i * 16 + g] = o[i][1];
    base[(2 * t) * HD + i * 16 + g + 8] = o[i][2];
    base[(2 * t + 1) * HD + i * 16 + g + 8] = o[i][3];
  }
  if (g == 0) {
    w_ml[(warp * GH + 2 * t) * 2] = m_run[0];
    w_ml[(warp * GH + 2 * t) * 2 + 1] = l_run[0];
    w_ml[(warp * GH + 2 * t + 1) * 2] = m_run[1];
    w_ml[(warp * GH + 2 * t + 1) * 2 + 1] = l_run[1];
  }
  __syncthreads();
  // merge the warps -> partial result of this split (maxima in units of log2 e)
  unsigned c_remote = 0;    // this split's place in split 0's shared memory
  if constexpr (clustered) {
    asm volatile("barrier.cluster.wait.aligned;\n" ::: "memory");
    const unsigned local = (unsigned)__cvta_generic_to_shared(c_part + (size_t)split * group * (HD + 2));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(c_remote) : "r"(local), "r"(0));
  }
  for (int i = tid; i < group * HD; i += NT) {
    const int gh = i / HD, c = i - gh * HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, w_ml[(w * GH + gh) * 2]);
    float a = 0.0f, l = 0.0f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float mw = w_ml[(w * GH + gh) * 2];
      const float f = (mw == -INFINITY) ? 0.0f : nb_exp2(mw - M);
      a += f * w_acc[(w * GH + gh) * HD + c];
      l += f * w_ml[(w * GH + gh) * 2 + 1];
    }
    const int head = kvh * group + gh;
    if (n_splits == 1) {
      out[(size_t)r * out_stride + (size_t)head * HD + c] = nb_from_f32<TOut>(l > 0.0f ? a / l : a);
      continue;
    }
    if constexpr (clustered) {
      const unsigned at = c_remote + (unsigned)(gh * (HD + 2)) * 4u;
      asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(at + (unsigned)c * 4u), "f"(a) : "memory");
      if (c == 0) {
        asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(at + (unsigned)HD * 4u), "f"(M) : "memory");
        asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(at + (unsigned)(HD + 1) * 4u), "f"(l) : "memory");
      }
      continue;
    }
    const size_t pi = ((size_t)r * n_heads + head) * n_splits + split;
    part_acc[pi * HD + c] = a;
    if (c == 0) {
      part_ml[pi * 2] = M;
      part_ml[pi * 2 + 1] = l;
    }
  }
  if (n_splits == 1) return;
  if constexpr (clustered) {
    // the stores above are visible to split 0 once every CTA has arrived (release) and split 0
    // has waited (acquire); the other splits wait too, so that none leaves the cluster early
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    if (split != 0) return;
    for (int i = tid; i < group * HD; i += NT) {
      const int gh = i / HD, c = i - gh * HD;
      const float* row = c_part + (size_t)gh * (HD + 2);
      const int step = group * (HD + 2);
      float M = -INFINITY;
      for (int s = 0; s < n_splits; ++s) M = fmaxf(M, row[s * step + HD]);
      float a = 0.0f, l = 0.0f;
      for (int s = 0; s < n_splits; ++s) {
        const float ms = row[s * step + HD];
        const float f = (ms == -INFINITY) ? 0.0f : nb_exp2(ms - M);
        a += f * row[s * step + c];
        l += f * row[s * step + HD + 1];
      }
      out[(size_t)r * out_stride + (size_t)(kvh * group + gh) * HD + c] =
          nb_from_f32<TOut>(l > 0.0f ? a / l : a);
    }
    return;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&counters[r * kv.n_kv_heads + kvh], 1);
    s_last = (old == n_splits - 1);
    if (s_last) counters[r * kv.n_kv_heads + kvh] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int i = tid; i < group * HD; i += NT) {
    const int gh = i / HD, c = i - gh * HD;
    const int head = kvh * group + gh;
    const size_t base = ((size_t)r * n_heads + head) * n_splits;
    // eight splits at a time, everything asked for before anything is used: one trip to L2
    // for the maxima, the sums and the partial results together
    float M = -INFINITY, a = 0.0f, l = 0.0f;
    for (int s0 = 0; s0 < n_splits; s0 += 8) {
      float2 ml8[8];
      float acc8[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool in = s0 + j < n_splits;
        ml8[j] = in ? __ldcg(reinterpret_cast<const float2*>(part_ml + (base + s0 + j) * 2))
                    : make_float2(-INFINITY, 0.0f);
        acc8[j] = in ? __ldcg(&part_acc[(base + s0 + j) * HD + c]) : 0.0f;
      }
      float Mn = M;
#pragma unroll
      for (int j = 0; j < 8; ++j) Mn = fmaxf(Mn, ml8[j].x);
      const float keep = (M == -INFINITY) ? 0.0f : nb_exp2(M - Mn);
      a *= keep;
      l *= keep;
#pragma unroll
      for (int j = 0; j < 8; ++j) {   // in split order
        const float f = (ml8[j].x == -INFINITY) ? 0.0f : nb_exp2(ml8[j].x - Mn);
        a += f * acc8[j];
        l += f * ml8[j].y;
      }
      M = Mn;
    }
    out[(size_t)r * out_stride + (size_t)head * HD + c] = nb_from_f32<TOut>(l > 0.0f ? a / l : a);
  }
}

template <int HD, typename TOut, int MMA_STAGES, int NW>
int launch_mma_s(const void* q, int q_stride, int q_col, const int* row_slot, const int* row_pos,
                 const NbPagedKV& kv, int group, void* out, int out_stride, float scale, int window,
                 int n_rows, int n_splits, float* part_acc, float* part_ml, int* counters, int append,
                 int k_col, int v_col, bool clustered, cudaStream_t stream) {
  const size_t tiles = (size_t)2 * MMA_STAGES * PAGE_TOKENS * (HD + 8) * sizeof(__nv_bfloat16);
  // room for the splits' partial results in split 0's shared memory (see the kernel)
  const size_t most = tiles + (size_t)MAX_CLUSTER * 8 * (HD + 2) * sizeof(float);
  dim3 grid(n_splits, kv.n_kv_heads, n_rows);
  if (clustered) {
    auto kern = attention_decode_mma_kernel<HD, TOut, MMA_STAGES, true, NW>;
    static bool configured = false;   // per instantiation
    if (most > 48 * 1024 && !configured) {
      NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most));
      configured = true;
    }
    const size_t smem = tiles + (size_t)n_splits * group * (HD + 2) * sizeof(float);
    NB_CUDA(nb_launch_clusters(kern, grid, dim3(NW * 32), smem, stream, n_splits,
                               (const __nv_bfloat16*)q, q_stride, q_col, row_slot, row_pos, kv, group,
                               (TOut*)out, out_stride, scale, window, n_splits, part_acc, part_ml,
                               counters, append, k_col, v_col));
    return 0;
  }
  auto kern = attention_decode_mma_kernel<HD, TOut, MMA_STAGES, false, NW>;
  static bool configured = false;   // per instantiation
  if (tiles > 48 * 1024 && !configured) {
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tiles));
    configured = true;
  }
  NB_CUDA(nb_launch(kern, grid, dim3(NW * 32), tiles, stream, (const __nv_bfloat16*)q, q_stride, q_col,
                    row_slot, row_pos, kv, group, (TOut*)out, out_stride, scale, window, n_splits,
                    part_acc, part_ml, counters, append, k_col, v_col));
  return 0;
}

template <int HD, typename TOut>
int launch_mma(const void* q, int q_stride, int q_col, const int* row_slot, const int* row_pos,
               const NbPagedKV& kv, int group, void* out, int out_stride, float scale, int window,
               int n_rows, int n_splits, float* part_acc, float* part_ml, int* counters, int append,
               int k_col, int v_col, bool clustered, cudaStream_t stream) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  // Eight warps and four pages in flight per CTA when the whole launch fits on the GPU that
  // way (an SM has 228 KB of shared memory, a CTA costs its own and 1 KB), else four warps and
  // two pages, for more CTAs per SM.
  const size_t smem4 = (size_t)8 * PAGE_TOKENS * (HD + 8) * sizeof(__nv_bfloat16) +
                       (clustered ? (size_t)n_splits * group * (HD + 2) * sizeof(float) : 0);
  const long long ctas = (long long)n_splits * kv.n_kv_heads * n_rows;
  long long per_sm = (long long)((228 * 1024) / (smem4 + 1024));
  if (per_sm > 8) per_sm = 8;   // 2,048 threads an SM
  if (ctas <= per_sm * sms)
    return launch_mma_s<HD, TOut, 4, 8>(q, q_stride, q_col, row_slot, row_pos, kv, group, out, out_stride,
                                        scale, window, n_rows, n_splits, part_acc, part_ml, counters,
                                        append, k_col, v_col, clustered, stream);
  return launch_mma_s<HD, TOut, 2, 4>(q, q_stride, q_col, row_slot, row_pos, kv, group, out, out_stride,
                                      scale, window, n_rows, n_splits, part_acc, part_ml, counters, append,
                                      k_col, v_col, clustered, stream);
}

template <typename TOut>
int mma_by_head_dim(int hd, const void* q, int q_stride, int q_col, const int* row_slot,
                    const int* row_pos, const NbPagedKV& kv, int group, void* out, int out_stride,
                    float scale, int window, int n_rows, int n_splits, float* pa, float* pm,
                    int* cn, int ap, int kc, int vc, bool clustered, cudaStream_t st) {
#define NB_HD(HD_) \
  case HD_: return launch_mma<HD_, TOut>(q, q_stride, q_col, row_slot, row_pos, kv, group, out, out_stride, scale, window, n_rows, n_splits, pa, pm, cn, ap, kc, vc, clustered, st)
  switch (hd) {
    NB_HD(16); NB_HD(32); NB_HD(48); NB_HD(64); NB_HD(80); NB_HD(96); NB_HD(112); NB_HD(128);
  }
#undef NB_HD
  return NB_ERR_UNSUPPORTED;
}

template <typename T, int HD, int G, typename TOut>
int launch(const void* q, int q_stride, int q_col, const int* row_slot, const int* row_pos,
           const NbPagedKV& kv, int group, void* out, int out_stride, float scale, int window,
           int n_rows, int n_splits, float* part_acc, float* part_ml, int* counters, int append,
           int k_col, int v_col, cudaStream_t stream) {
  const size_t smem = (size_t)4 * PAGE_TOKENS * HD * sizeof(T) +
                      (size_t)(G * HD + WARPS * G * HD + WARPS * G * 2) * sizeof(float);
  auto kern = attention_decode_kernel<T, HD, G, TOut>;
  if (smem > 48 * 1024)
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(n_splits, kv.n_kv_heads, n_rows);
  NB_CUDA(nb_launch(kern, grid, dim3(THREADS), smem, stream, (const T*)q, q_stride, q_col, row_slot,
                    row_pos, kv, group, (TOut*)out, out_stride, scale, window, n_splits, part_acc,
                    part_ml, counters, append, k_col, v_col));
  return 0;
}

template <typename T, int HD, typename TOut>
int by_group(int group, const void* q, int q_stride, int q_col, const int* row_slot,
             const int* row_pos, const NbPagedKV& kv, void* out, int out_stride, float scale,
             int window, int n_rows, int n_splits, float* pa, float* pm, int* cn, int ap,
             int kc, int vc, cudaStream_t st) {
#define NB_G(G_) \
  return launch<T, HD, G_, TOut>(q, q_stride, q_col, row_slot, row_pos, kv, group, out, out_stride, scale, window, n_rows, n_splits, pa, pm, cn, ap, kc, vc, st)
  if (group == 1) NB_G(1);
  if (group == 2) NB_G(2);
  if (group <= 4) NB_G(4);
  NB_G(8);
#undef NB_G
}

template <typename T, typename TOut>
int by_head_dim(int hd, int group, const void* q, int q_stride, int q_col, const int* row_slot,
                const int* row_pos, const NbPagedKV& kv, void* out, int out_stride, float scale,
                int window, int n_rows, int n_splits, float* pa, float* pm, int* cn, int ap,
                int kc, int vc, cudaStream_t st) {
#define NB_HD(HD_) \
  return by_group<T, HD_, TOut>(group, q, q_stride, q_col, row_slot, row_pos, kv, out, out_stride, scale, window, n_rows, n_splits, pa, pm, cn, ap, kc, vc, st)
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

// 1 if this kernel takes the shape (otherwise the caller uses the generic kernel).
NB_EXPORT int nb_attention_decode_supported(int dtype, int head_dim, int n_heads, int n_kv_heads,
                                            int page) {
  if (page != PAGE_TOKENS || n_kv_heads < 1 || n_heads % n_kv_heads != 0) return 0;
  if (n_heads / n_kv_heads > 8) return 0;
  if (dtype == NB_BF16) return head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 128;
  if (dtype != NB_F32) return 0;
  return head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128;
}

// Floats of part_acc, floats of part_ml and ints of counters that a launch needs.
NB_EXPORT void nb_attention_decode_scratch(int n_rows, int n_heads, int n_kv_heads, int head_dim,
                                           int n_splits, long long* acc_floats,
                                           long long* ml_floats, long long* counter_ints) {
  *acc_floats = (long long)n_rows * n_heads * n_splits * head_dim;
  *ml_floats = (long long)n_rows * n_heads * n_splits * 2;
  *counter_ints = (long long)n_rows * n_kv_heads;
}

// append != 0: row r of `q` also holds this step's key and value at columns k_col / v_col;
// the kernel writes them to the cache at token row_pos[r] and attends to them as well, so no
// separate append pass is needed.
namespace {
std::atomic<int> g_cluster_merge{1};

int attention_decode(const void* q, int dtype, int q_stride, int q_col, const int* row_slot,
                     const int* row_pos, const void* k_cache, const void* v_cache,
                     const int* block_table, int max_pages, int page, int n_heads, int n_kv_heads,
                     int head_dim, void* out, int out_dtype, int out_stride, float scale, int window,
                     int n_rows, int n_splits, float* part_acc, float* part_ml, int* counters,
                     int append, int k_col, int v_col, int clusters_allowed, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(nb_attention_decode_supported(dtype, head_dim, n_heads, n_kv_heads, page),
             NB_ERR_UNSUPPORTED,
             "attention_decode: unsupported shape (head size %d, %d/%d heads, page %d)", head_dim,
             n_heads, n_kv_heads, page);
  NB_REQUIRE(n_splits >= 1 && n_splits <= 65535 && n_rows <= 65535 && n_kv_heads <= 65535,
             NB_ERR_UNSUPPORTED, "attention_decode: grid too large");
  NB_REQUIRE(part_acc && part_ml && counters, NB_ERR_BAD_ARG, "attention_decode: scratch missing");
  if (append) {
    const int epl = dtype == NB_F32 ? 4 : 8;
    NB_REQUIRE(q_stride % epl == 0 && k_col % epl == 0 && v_col % epl == 0 && (uintptr_t)q % 16 == 0,
               NB_ERR_UNSUPPORTED, "attention_decode: keys/values to append must be 16-byte aligned");
  }
  NbPagedKV kv{(void*)k_cache, (void*)v_cache, block_table, max_pages, page, n_kv_heads, head_dim};
  const int group = n_heads / n_kv_heads;
  typedef __nv_bfloat16 bf16;
  int rc;
#define NB_ARGS head_dim, group, q, q_stride, q_col, row_slot, row_pos, kv, out, out_stride, scale, window, n_rows, n_splits, part_acc, part_ml, counters, append, k_col, v_col, stream
  if (dtype == NB_F32) {
    rc = out_dtype == NB_F32 ? by_head_dim<float, float>(NB_ARGS) : by_head_dim<float, bf16>(NB_ARGS);
  } else {
    // bf16 cache: tensor cores (needs 16-byte aligned rows and 4-byte aligned query columns)
    NB_REQUIRE(q_stride % 8 == 0 && q_col % 2 == 0 && (uintptr_t)q % 16 == 0, NB_ERR_UNSUPPORTED,
               "attention_decode: query rows must be 16-byte aligned");
    // up to MAX_CLUSTER splits merge through the shared memory of a thread-block cluster, more
    // through the scratch arrays and a counter
    const bool clustered = clusters_allowed > 0 && n_splits >= 2 && n_splits <= MAX_CLUSTER;
    rc = out_dtype == NB_F32
             ? mma_by_head_dim<float>(head_dim, q, q_stride, q_col, row_slot, row_pos, kv, group, out, out_stride, scale, window, n_rows, n_splits, part_acc, part_ml, counters, append, k_col, v_col, clustered, stream)
             : mma_by_head_dim<bf16>(head_dim, q, q_stride, q_col, row_slot, row_pos, kv, group, out, out_stride, scale, window, n_rows, n_splits, part_acc, part_ml, counters, append, k_col, v_col, clustered, stream);
  }
#undef NB_ARGS
  if (rc) return rc;
  NB_CHECK_LAUNCH("attention_decode");
  return 0;
}
}  // namespace

NB_EXPORT int nb_attention_decode(const void* q, int dtype, int q_stride, int q_col,
                                  const int* row_slot, const int* row_pos, const void* k_cache,
                                  const void* v_cache, const int* block_table, int max_pages,
                                  int page, int n_heads, int n_kv_heads, int head_dim, void* out,
                                  int out_dtype, int out_stride, float scale, int window,
                                  int n_rows, int n_splits, float* part_acc, float* part_ml,
                                  int* counters, int append, int k_col, int v_col,
                                  cudaStream_t stream) {
  return attention_decode(q, dtype, q_stride, q_col, row_slot, row_pos, k_cache, v_cache, block_table,
                          max_pages, page, n_heads, n_kv_heads, head_dim, out, out_dtype, out_stride,
                          scale, window, n_rows, n_splits, part_acc, part_ml, counters, append, k_col,
                          v_col, g_cluster_merge.load(), stream);
}

// How the splits of the bfloat16 kernel merge: 0 always through the scratch arrays; otherwise
// (the default) through a cluster's shared memory where there are 2 to 8 of them.  Returns the
// earlier setting.
NB_EXPORT int nb_attention_decode_cluster_merge(int mode) {
  return g_cluster_merge.exchange(mode != 0 ? 1 : 0);
}

// Most splits that merge inside a cluster.
NB_EXPORT int nb_attention_decode_cluster_limit() { return MAX_CLUSTER; }

// ---------------------------------------------------------------------------------------
// The same kernel for callers that cannot allocate device memory (see no_alloc.h).
// Its scratch is this file-scope array: every GPU that loads the library holds these
// NB_STATIC_SCRATCH_BYTES until the process exits.
// ---------------------------------------------------------------------------------------
#include "no_alloc.h"

static __device__ __align__(256) unsigned char g_static_scratch[NB_STATIC_SCRATCH_BYTES];

namespace {
constexpr int MAX_DEVICES = 64;
std::mutex g_static_mutex;
void* g_static_ptr[MAX_DEVICES] = {nullptr};

// The array's device address on the current device.  In host code the name
// `g_static_scratch` is only a handle for the runtime, never an address a kernel may use.
int static_scratch_address(unsigned char** out, cudaStream_t stream) {
  int dev = -1;
  NB_CUDA(cudaGetDevice(&dev));
  NB_REQUIRE(dev >= 0 && dev < MAX_DEVICES, NB_ERR_UNSUPPORTED,
             "attention_decode_static: device index %d is beyond %d", dev, MAX_DEVICES);
  // the address below is the current device's copy of the array: a stream of another device
  // would run the kernel there, on memory it does not own
  int stream_dev = dev;
  if (stream != nullptr && cudaStreamGetDevice(stream, &stream_dev) != cudaSuccess) {
    (void)cudaGetLastError();
    stream_dev = dev;
  }
  NB_REQUIRE(stream_dev == dev, NB_ERR_BAD_ARG,
             "attention_decode_static: the stream belongs to device %d, the current device is %d",
             stream_dev, dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    NB_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    NB_REQUIRE(p != nullptr, NB_ERR_UNSUPPORTED, "attention_decode_static: no symbol address");
    g_static_ptr[dev] = p;
  }
  *out = static_cast<unsigned char*>(g_static_ptr[dev]);
  return 0;
}
}  // namespace

NB_EXPORT long long nb_attention_decode_static_capacity() { return NB_STATIC_SCRATCH_BYTES; }

NB_EXPORT int nb_attention_decode_static(const void* q, int dtype, int q_stride, int q_col,
                                         const int* row_slot, const int* row_pos,
                                         const void* k_cache, const void* v_cache,
                                         const int* block_table, int max_pages, int page,
                                         int n_heads, int n_kv_heads, int head_dim, void* out,
                                         int out_dtype, int out_stride, float scale, int window,
                                         int n_rows, int n_splits, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(n_rows > 0 && n_heads > 0 && n_kv_heads > 0 && head_dim > 0 && n_splits > 0,
             NB_ERR_BAD_ARG, "attention_decode_static: sizes must be positive");
  long long acc_f = 0, ml_f = 0, cnt_i = 0;
  nb_attention_decode_scratch(n_rows, n_heads, n_kv_heads, head_dim, n_splits, &acc_f, &ml_f, &cnt_i);
  // layout: [counters | (max,sum) pairs | partial sums], each part rounded up to 256 bytes
  auto up = [](long long b) { return (b + 255) / 256 * 256; };
  const long long cnt_b = up(cnt_i * 4), ml_b = up(ml_f * 4), acc_b = up(acc_f * 4);
  NB_REQUIRE(cnt_b + ml_b + acc_b <= (long long)NB_STATIC_SCRATCH_BYTES, NB_ERR_UNSUPPORTED,
             "attention_decode_static: %d rows x %d heads x %d splits x head size %d need %lld "
             "bytes of scratch, the built-in array holds %lld; use fewer splits or "
             "nb_attention_decode with scratch of your own",
             n_rows, n_heads, n_splits, head_dim, cnt_b + ml_b + acc_b,
             (long long)NB_STATIC_SCRATCH_BYTES);
  unsigned char* base = nullptr;
  const int rc = static_scratch_address(&base, stream);
  if (rc) return rc;
  // the array keeps what the last call left; the counters are the only part that must start
  // at zero (a launch that ran to its end leaves them so, an interrupted one may not)
  NB_CUDA(cudaMemsetAsync(base, 0, (size_t)cnt_b, stream));
  // always through the scratch arrays: this entry point exists for them
  return attention_decode(q, dtype, q_stride, q_col, row_slot, row_pos, k_cache, v_cache,
                          block_table, max_pages, page, n_heads, n_kv_heads, head_dim, out,
                          out_dtype, out_stride, scale, window, n_rows, n_splits,
                          reinterpret_cast<float*>(base + cnt_b + ml_b),
                          reinterpret_cast<float*>(base + cnt_b),
                          reinterpret_cast<int*>(base), /*append=*/0, 0, 0,
                          /*clusters_allowed=*/0, stream);
}
