// Prefill attention: many query rows per sequence over the paged key/value cache, bf16 on the
// tensor cores with fp32 softmax (running maximum and sum per row, probabilities rounded to
// bf16 only as the operand of the value product).
//
// One CTA takes 64 consecutive query rows of one sequence and one head; each of its four warps
// owns 16 rows.  Key/value pages (64 tokens x head_dim, contiguous in the cache) are streamed
// into shared memory with cp.async, two pages in flight; scores are mma.sync m16n8k16 products
// of the query fragments (held in registers) with the page's keys, the causal limit (and the
// window) is applied to the fp32 scores, and the probabilities, re-used in place as the next
// product's A operand, multiply the page's values.  Rows of a sequence sit anywhere in the
// packed batch (cu_rows) and start at any cached length (seq_pos0), so chunks that continue a
// sequence work like whole prompts.
//
// This kernel uses the legacy mma.sync tensor-core path, not tcgen05.
//
// Reference: src/model.rs:401-422 (scores = dot(q,k)*scale for keys 0..P+i, softmax with the
// maximum subtracted, weighted values).
#include "attention_common.cuh"

namespace {

typedef __nv_bfloat16 bf16;
constexpr int THREADS = 128;
constexpr int BLOCK_Q = 64;
constexpr int PAGE_TOKENS = 64;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <int HD, typename TOut>
__global__ void __launch_bounds__(THREADS)
attention_prefill_kernel(const bf16* __restrict__ q, int q_stride, int q_col,
                         const int* __restrict__ cu_rows, const int* __restrict__ seq_slot,
                         const int* __restrict__ seq_pos0, NbPagedKV kv, int group,
                         TOut* __restrict__ out, int out_stride, float scale, int window) {
  constexpr int ROW = HD + 8;              // padded row (elements): ldmatrix without conflicts
  constexpr int KS = HD / 16;              // k-steps of the score product
  constexpr int NT = HD / 8;               // n-tiles of the value product
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);          // [64][ROW]
  bf16* kv_s = q_s + BLOCK_Q * ROW;                        // [2 stages][K | V][64][ROW]

  const int tile = blockIdx.x, h = blockIdx.y, s = blockIdx.z;
  const int row0 = cu_rows[s], n_q = cu_rows[s + 1] - row0;
  const int q0 = tile * BLOCK_Q;
  if (q0 >= n_q) return;
  const int slot = seq_slot[s];
  if (slot < 0) return;
  const int pos0 = seq_pos0[s];
  const int kvh = h / group;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rows_here = min(BLOCK_Q, n_q - q0);
  const int last_pos = pos0 + q0 + rows_here - 1;                    // newest key any row sees
  const int first_key = (window > 0) ? max(0, pos0 + q0 + 1 - window) : 0;
  const int p_begin = first_key / PAGE_TOKENS, p_end = last_pos / PAGE_TOKENS + 1;
  const int* table = kv.block_table + (size_t)slot * kv.max_pages;

  auto issue = [&](int page_idx, int stage) {
    const int page_id = table[page_idx];
    const bf16* ksrc = (const bf16*)kv.k + ((size_t)page_id * kv.n_kv_heads + kvh) * PAGE_TOKENS * HD;
    const bf16* vsrc = (const bf16*)kv.v + ((size_t)page_id * kv.n_kv_heads + kvh) * PAGE_TOKENS * HD;
    bf16* kdst = kv_s + (size_t)stage * 2 * PAGE_TOKENS * ROW;
    bf16* vdst = kdst + PAGE_TOKENS * ROW;
    constexpr int CPR = HD / 8;   // 16-byte chunks per row
    for (int i = tid; i < PAGE_TOKENS * CPR; i += THREADS) {
      const int r = i / CPR, c = i - r * CPR;
      cp_async16(kdst + r * ROW + c * 8, ksrc + r * HD + c * 8);
      cp_async16(vdst + r * ROW + c * 8, vsrc + r * HD + c * 8);
    }
    cp_async_commit();
  };
  issue(p_begin, 0);

  // the query tile: rows beyond the sequence are zero
  {
    constexpr int CPR = HD / 8;
    for (int i = tid; i < BLOCK_Q * CPR; i += THREADS) {
      const int r = i / CPR, c = i - r * CPR;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < rows_here)
        v = *reinterpret_cast<const uint4*>(q + (size_t)(row0 + q0 + r) * q_stride + q_col +
                                            (size_t)h * HD + c * 8);
      *reinterpret_cast<uint4*>(q_s + r * ROW + c * 8) = v;
    }
  }
  __syncthreads();
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks)
    ldmatrix_x4(qf[ks], q_s + (warp * 16 + (lane & 15)) * ROW + ks * 16 + (lane >> 4) * 8);

  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[n][j] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  const float sl2 = scale * 1.4426950408889634f;    // scores in units of log2(e)
  const int qpos_a = pos0 + q0 + warp * 16 + g;     // absolute position of row g
  const int qpos_b = qpos_a + 8;                    // ... and of row g + 8

  for (int p = p_begin; p < p_end; ++p) {
    const int stage = (p - p_begin) & 1;
    if (p + 1 < p_end) {
      issue(p + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* kt = kv_s + (size_t)stage * 2 * PAGE_TOKENS * ROW;
    bf16* vt = kv_s + (size_t)stage * 2 * PAGE_TOKENS * ROW + PAGE_TOKENS * ROW;
    // Rows of the last page after the newest key hold whatever an earlier owner of the page
    // left there.  Their probabilities are zero, but zero times a non-finite value is not: the
    // value rows are cleared in the staged copy (masked scores are replaced, not multiplied).
    const int tail_row = last_pos + 1 - p * PAGE_TOKENS;
    if (tail_row < PAGE_TOKENS) {   // uniform over the CTA
      constexpr int CPR = HD / 8;
      for (int i = tid; i < (PAGE_TOKENS - tail_row) * CPR; i += THREADS) {
        const int r = tail_row + i / CPR, c = (i % CPR) * 8;
        *reinterpret_cast<uint4*>(vt + r * ROW + c) = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncthreads();
    }

    // scores of 16 rows x 64 keys
    float sc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) sc[n][j] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int n2 = 0; n2 < 4; ++n2) {   // two key tiles of 8 per ldmatrix.x4
        uint32_t kb[4];
        ldmatrix_x4(kb, kt + (n2 * 16 + (lane & 7) + (lane >> 4) * 8) * ROW + ks * 16 +
                            ((lane >> 3) & 1) * 8);
        mma_bf16(sc[2 * n2], qf[ks], kb[0], kb[1]);
        mma_bf16(sc[2 * n2 + 1], qf[ks], kb[2], kb[3]);
      }
    }
    // causal limit, window, scale; running maximum.  A page that lies wholly before the first
    // row of this warp (and needs no window) is visible to all of its rows: no comparisons.
    const int j0 = p * PAGE_TOKENS;
    float mx[2] = {-INFINITY, -INFINITY};
    if (window <= 0 && j0 + PAGE_TOKENS - 1 <= pos0 + q0 + warp * 16) {
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float v = sc[n][j] * sl2;
          sc[n][j] = v;
          mx[j >> 1] = fmaxf(mx[j >> 1], v);
        }
      }
    } else {
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int key = j0 + n * 8 + t * 2 + (j & 1);
          const int qp = (j < 2) ? qpos_a : qpos_b;
          const bool ok = key <= qp && (window <= 0 || key > qp - window);
          const float v = ok ? sc[n][j] * sl2 : -INFINITY;
          sc[n][j] = v;
          mx[j >> 1] = fmaxf(mx[j >> 1], v);
        }
      }
    }
    float m_use[2], resc[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = (m_new == -INFINITY) ? 0.0f : m_new;
      resc[r] = (m_run[r] == -INFINITY) ? 0.0f : nb_exp2(m_run[r] - m_use[r]);
      m_run[r] = m_new;
      l_run[r] *= resc[r];
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      o[n][0] *= resc[0]; o[n][1] *= resc[0];
      o[n][2] *= resc[1]; o[n][3] *= resc[1];
    }
    // probabilities (fp32), their row sums, and their bf16 form as the next A operand
    uint32_t pf[4][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const float p0 = nb_exp2(sc[n][0] - m_use[0]), p1 = nb_exp2(sc[n][1] - m_use[0]);
      const float p2 = nb_exp2(sc[n][2] - m_use[1]), p3 = nb_exp2(sc[n][3] - m_use[1]);
      l_run[0] += p0 + p1;
      l_run[1] += p2 + p3;
      pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
      pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    // o += P V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {       // 16 keys per step
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2) {   // two value tiles of 8 columns per ldmatrix.x4
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ROW + n2 * 16 +
                                  (lane >> 4) * 8);
        mma_bf16(o[2 * n2], pf[kk], vb[0], vb[1]);
        mma_bf16(o[2 * n2 + 1], pf[kk], vb[2], vb[3]);
      }
    }
    __syncthreads();   // the stage may be refilled
  }

  // row sums across the four lanes of a row, then the result
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  const float inv_a = l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f;
  const float inv_b = l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f;
  const int ra = warp * 16 + g, rb = ra + 8;
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int col = h * HD + n * 8 + t * 2;
    if (ra < rows_here) {
      TOut* dst = out + (size_t)(row0 + q0 + ra) * out_stride + col;
      dst[0] = nb_from_f32<TOut>(o[n][0] * inv_a);
      dst[1] = nb_from_f32<TOut>(o[n][1] * inv_a);
    }
    if (rb < rows_here) {
      TOut* dst = out + (size_t)(row0 + q0 + rb) * out_stride + col;
      dst[0] = nb_from_f32<TOut>(o[n][2] * inv_b);
      dst[1] = nb_from_f32<TOut>(o[n][3] * inv_b);
    }
  }
}

template <int HD, typename TOut>
int launch(const void* q, int q_stride, int q_col, const int* cu_rows, const int* seq_slot,
           const int* seq_pos0, const NbPagedKV& kv, int n_heads, void* out, int out_stride,
           float scale, int window, int n_seqs, int max_q_len, cudaStream_t stream) {
  constexpr int ROW = HD + 8;
  const size_t smem = (size_t)(BLOCK_Q + 4 * PAGE_TOKENS) * ROW * sizeof(bf16);
  auto kern = attention_prefill_kernel<HD, TOut>;
  if (smem > 48 * 1024)
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((max_q_len + BLOCK_Q - 1) / BLOCK_Q, n_heads, n_seqs);
  kern<<<grid, THREADS, smem, stream>>>((const bf16*)q, q_stride, q_col, cu_rows, seq_slot,
                                        seq_pos0, kv, n_heads / kv.n_kv_heads, (TOut*)out,
                                        out_stride, scale, window);
  return 0;
}

}  // namespace

NB_EXPORT int nb_attention_prefill_supported(int dtype, int head_dim, int n_heads, int n_kv_heads,
                                             int page, int q_stride, int q_col) {
  if (dtype != NB_BF16 || page != PAGE_TOKENS) return 0;
  if (n_kv_heads < 1 || n_heads % n_kv_heads != 0) return 0;
  if (q_stride % 8 != 0 || q_col % 8 != 0) return 0;   // 16-byte query loads
  return head_dim == 16 || head_dim == 32 || head_dim == 48 || head_dim == 64 ||
         head_dim == 96 || head_dim == 128;
}

// Rows of sequence s are cu_rows[s]..cu_rows[s+1] of the packed batch, at positions
// seq_pos0[s].. of slot seq_slot[s]; their keys and values are already in the cache.
NB_EXPORT int nb_attention_prefill(const void* q, int dtype, int q_stride, int q_col,
                                   const int* cu_rows, const int* seq_slot, const int* seq_pos0,
                                   const void* k_cache, const void* v_cache,
                                   const int* block_table, int max_pages, int page, int n_heads,
                                   int n_kv_heads, int head_dim, void* out, int out_dtype,
                                   int out_stride, float scale, int window, int n_seqs,
                                   int max_q_len, cudaStream_t stream) {
  if (n_seqs == 0 || max_q_len == 0) return 0;
  NB_REQUIRE(nb_attention_prefill_supported(dtype, head_dim, n_heads, n_kv_heads, page, q_stride, q_col),
             NB_ERR_UNSUPPORTED,
             "attention_prefill: unsupported shape (head size %d, %d/%d heads, row pitch %d)",
             head_dim, n_heads, n_kv_heads, q_stride);
  NB_REQUIRE(n_seqs <= 65535 && n_heads <= 65535, NB_ERR_UNSUPPORTED,
             "attention_prefill: grid too large");
  NB_REQUIRE((uintptr_t)q % 16 == 0, NB_ERR_UNSUPPORTED, "attention_prefill: unaligned queries");
  NbPagedKV kv{(void*)k_cache, (void*)v_cache, block_table, max_pages, page, n_kv_heads, head_dim};
  int rc = NB_ERR_UNSUPPORTED;
#define NB_HD(HD_)                                                                             \
  case HD_:                                                                                    \
    rc = out_dtype == NB_F32                                                                   \
             ? launch<HD_, float>(q, q_stride, q_col, cu_rows, seq_slot, seq_pos0, kv, n_heads, out, out_stride, scale, window, n_seqs, max_q_len, stream) \
             : launch<HD_, bf16>(q, q_stride, q_col, cu_rows, seq_slot, seq_pos0, kv, n_heads, out, out_stride, scale, window, n_seqs, max_q_len, stream); \
    break;
  switch (head_dim) {
    NB_HD(16) NB_HD(32) NB_HD(48) NB_HD(64) NB_HD(96) NB_HD(128)
  }
#undef NB_HD
  if (rc) return rc;
  NB_CHECK_LAUNCH("attention_prefill");
  return 0;
}
