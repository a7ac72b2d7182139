// Prefill attention on the 5th-generation tensor cores (sm_100a): many query rows per
// sequence over the paged key/value cache, head size 64 or 128, bf16 operands, fp32 scores and
// softmax.
//
// One CTA takes 128 consecutive query rows of one sequence and one head; a row of the tile is
// a lane of tensor memory.  Warp 0 is the producer: one thread brings the query tile and then,
// two pages (128 keys) at a time, the pages' keys and values into a ring of shared-memory
// stages with TMA (the cache is [page][kv_head][64][head_dim], so a page of one head is a
// 64 x head_dim matrix that a tensor map addresses by its first row).  Warp 1 issues the
// products: S = Q K^T (tcgen05.mma, M=128, N=128, K=head_dim) into one of two score buffers
// in tensor memory, and O_j = P_j V_j (M=128, N=head_dim, K=128) into one of two output
// buffers; P_j is read from tensor memory, where the softmax wrote it over the scores it came
// from, and V is the MN-major operand, straight from its page layout.  With `append`, the
// step's own keys and values are not in the cache yet: pages at or after a sequence's cached
// length (a multiple of the page size) are read from the step's rows instead, and the CTA
// whose query rows a page belongs to copies it from shared memory into the cache with a TMA
// store (one CTA per key/value head).  Warps 2..9 are the
// softmax, two threads per row (one of the two pages and half of the head's columns each; a
// run of an odd number of pages ends with a turn of one page): a thread reads its scores with
// tcgen05.ld, applies scale, causal limit and window, keeps the running maximum and sum in
// fp32, writes the probabilities as bf16 back with tcgen05.st, and adds an earlier page's
// O_j, rescaled, to its fp32 outputs in registers.  The score product of turn j+1 runs while
// turn j is in the softmax.
//
// Every wait on an mbarrier is bounded by a clock budget; a wait that runs out raises an error
// flag (nb_attention_prefill_tc_error), all roles leave their loops, and the CTA frees its
// tensor memory and returns.
//
// Reference: src/model.rs:401-422 (scores = dot(q,k)*scale for keys 0..P+i, softmax with the
// maximum subtracted, weighted values).
#include "attention_common.cuh"
#include "tc05_common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

constexpr int TILE_Q = 128;
constexpr int PAGE_TOKENS = 64;
constexpr int TC_THREADS = 320;   // producer, MMA issuer, eight softmax warps


// kind::f16 instruction descriptor with an MN-major B operand (bit 16)
__host__ __device__ constexpr uint32_t instr_desc_bf16_b_mn(int m, int n) {
  return instr_desc_bf16(m, n) | (1u << 16);
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// D (tensor memory) = A (tensor memory, bf16 packed two per column) * B (shared memory)
__device__ __forceinline__ void tc05_mma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                                     uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc05_st_32x32b_x32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, "
      "%21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
      "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
      "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tc05_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}

template <int HD>
struct AttnSmem {
  static constexpr int HB = HD / 64;                      // 64-column boxes per row of a head
  static constexpr int Q_BYTES = TILE_Q * 128 * HB;       // [HB][128 rows][128 B]
  static constexpr int PAGE_BOX = PAGE_TOKENS * 128;      // one page, 64 head columns: 8 KB
  static constexpr int K_BYTES = 2 * PAGE_BOX * HB;       // [HB][2 pages][64 keys][128 B]
  static constexpr int V_BYTES = K_BYTES;
  static constexpr int STAGE_BYTES = K_BYTES + V_BYTES;
  static constexpr int STAGES = HD == 64 ? 4 : 2;         // 144 KB / 160 KB of tiles
  static constexpr int TILES_BYTES = Q_BYTES + STAGES * STAGE_BYTES;
  // q_full, kv_full[S], kv_empty[S], s_full[2], p_full[2], o_full[2], o_empty[2]
  static constexpr int N_BARRIERS = 1 + 2 * STAGES + 8;
  static constexpr int XCH_BYTES = 6 * TILE_Q * 4;   // row maxima (two buffers) and sums of the two halves
  static constexpr int TOTAL = TILES_BYTES + N_BARRIERS * 8 + 16 + XCH_BYTES + 1024 /* alignment slack */;
  // tensor memory columns: two score buffers of 128 (the probabilities of a turn take the
  // first 64 columns of its score buffer), two output buffers of HD
  static constexpr int S_COL = 0, O_COL = 256;
  static constexpr int TMEM_COLS = 512;
};

template <int HD, typename TOut>
__global__ void __launch_bounds__(TC_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                            const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v,
                            const __grid_constant__ CUtensorMap map_new, int append, int k_col,
                            int v_col, int q_col,
                            const int* cu_rows, const int* seq_slot,
                            const int* seq_pos0, const int* block_table,
                            int max_pages, int n_kv_heads, int group, TOut* out,
                            int out_stride, float scale, int window, int max_splits,
                            int chunk_pages, float* part, int* counters,
                            int* err_word) {
  using L = AttnSmem<HD>;
  constexpr int HB = L::HB;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gen = smem_dyn + (base - raw);
  const uint32_t q_smem = base;
  const uint32_t kv_smem = base + L::Q_BYTES;
  const uint32_t bars = base + L::TILES_BYTES;
  const uint32_t q_full = bars;
  auto kv_full = [&](int s) { return bars + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bars + 8u * (1 + L::STAGES + s); };
  auto s_full = [&](int b) { return bars + 8u * (1 + 2 * L::STAGES + b); };
  auto p_full = [&](int b) { return bars + 8u * (1 + 2 * L::STAGES + 2 + b); };
  auto o_full = [&](int b) { return bars + 8u * (1 + 2 * L::STAGES + 4 + b); };
  auto o_empty = [&](int b) { return bars + 8u * (1 + 2 * L::STAGES + 6 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + L::TILES_BYTES + L::N_BARRIERS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xch = reinterpret_cast<float*>(tmem_slot + 4);   // [2 buffers + sums][2 halves][128 rows]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // CTAs start in the order of their linear index.  That order is made "all heads and
  // sequences of the last tile, then of the tile before it, ...": the long tiles (late query
  // rows see many keys) start first, each on an SM of its own, and the short ones fill in
  // beside them at the end.
  const int linear = (int)blockIdx.x + (int)gridDim.x * ((int)blockIdx.y + (int)gridDim.y * (int)blockIdx.z);
  const int per_unit = (int)gridDim.y * (int)gridDim.z;
  const int unit = (int)gridDim.x - 1 - linear / per_unit;
  const int h = (linear % per_unit) % (int)gridDim.y, s = (linear % per_unit) / (int)gridDim.y;
  const int tile = unit / max_splits, split = unit % max_splits;
  const int row0 = cu_rows[s], n_q = cu_rows[s + 1] - row0;
  const int q0 = tile * TILE_Q;
  const int slot = seq_slot[s];
  // (a CTA that leaves waits for the kernel before this one all the same: a grid that ended
  // early would let the kernel after it overtake that one)
  if (q0 >= n_q || slot < 0) {                // the whole CTA leaves: nothing is allocated yet
    nb_grid_dependency_wait();
    return;
  }
  const int pos0 = seq_pos0[s];
  const int kvh = h / group;
  const int rows_here = min(TILE_Q, n_q - q0);
  const int last_pos = pos0 + q0 + rows_here - 1;                    // newest key any row sees
  const int first_key = (window > 0) ? max(0, pos0 + q0 + 1 - window) : 0;
  // The pages this tile reads are cut into runs of chunk_pages, one CTA each (the long tiles of
  // a short batch would otherwise be a few long serial chains); the CTAs of a tile leave their
  // partial results in `part`, and the one that finishes last adds them up.
  const int p_first = first_key / PAGE_TOKENS, p_last = last_pos / PAGE_TOKENS + 1;
  const int n_splits = (p_last - p_first + chunk_pages - 1) / chunk_pages;
  if (split >= n_splits) {
    nb_grid_dependency_wait();
    return;
  }
  const int p_begin = p_first + split * chunk_pages, p_end = min(p_last, p_begin + chunk_pages);
  const int nb = (p_end - p_begin + 1) / 2;             // turns of two pages
  const int tail_row = last_pos % PAGE_TOKENS + 1;      // first row of the last page without a key
  // turn i takes pages p_begin + 2i and, if it is still in the run, the next one
  auto two_pages = [&](int i) { return p_begin + 2 * i + 1 < p_end; };
  const int* table = block_table + (size_t)slot * max_pages;

  if (tid == 0) {
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
    if (append) prefetch_tensormap(&map_new);
    mbar_init(q_full, 1);
    for (int i = 0; i < L::STAGES; ++i) {
      mbar_init(kv_full(i), 1);
      mbar_init(kv_empty(i), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_full(b), 1);
      mbar_init(p_full(b), 8);     // one arrival per softmax warp
      mbar_init(o_full(b), 1);
      mbar_init(o_empty(b), 8);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"((uint32_t)L::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc05_fence_before();
  __syncthreads();
  tc05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // The batch layout and the block table are older than the kernel before this one; the rows
  // of queries, keys and values are its work.  Under a programmatic launch everything above
  // ran while it was finishing.
  nb_grid_dependency_wait();

  if (warp == 0) {
    if (lane == 0) {   // ------------------------------------------------------ TMA producer
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int b = 0; b < HB; ++b)
        tma_load_2d(q_smem + b * (TILE_Q * 128), &map_q, q_col + h * HD + b * 64, row0 + q0, q_full);
      bool ok = true;
      // keys and values of page p of the sequence, 64 head columns at a time: from the cache,
      // or (append) from the step's own rows when the page lies at or after the cached length
      auto load_page = [&](int p, int page_id, uint32_t kb, uint32_t vb, int b, uint32_t bar) {
        if (append && p * PAGE_TOKENS >= pos0) {
          const int row = row0 + p * PAGE_TOKENS - pos0;
          tma_load_2d(kb, &map_new, k_col + kvh * HD + b * 64, row, bar);
          tma_load_2d(vb, &map_new, v_col + kvh * HD + b * 64, row, bar);
        } else {
          const int row = (page_id * n_kv_heads + kvh) * PAGE_TOKENS;
          tma_load_2d(kb, &map_k, b * 64, row, bar);
          tma_load_2d(vb, &map_v, b * 64, row, bar);
        }
      };
      // (append) a page of this tile's own query rows goes from shared memory into the cache
      const bool writer = append && (h % group == 0);
      bool stored = false;
      auto store_page = [&](int p, int page_id, uint32_t kb, uint32_t vb, int b) {
        if (p * PAGE_TOKENS < pos0 + q0) return;
        const int row = (page_id * n_kv_heads + kvh) * PAGE_TOKENS;
        tma_store_2d(&map_k, kb, b * 64, row);
        tma_store_2d(&map_v, vb, b * 64, row);
        stored = true;
      };
      int next_a = table[p_begin];
      int next_b = two_pages(0) ? table[p_begin + 1] : 0;
      for (int j = 0; j < nb && ok; ++j) {
        const int st = j % L::STAGES;
        const int page_a = next_a, page_b = next_b;
        const bool two = two_pages(j);
        if (j + 1 < nb) {
          next_a = table[p_begin + 2 * j + 2];
          next_b = two_pages(j + 1) ? table[p_begin + 2 * j + 3] : 0;
        }
        ok = mbar_wait(kv_empty(st), ((j / L::STAGES) & 1u) ^ 1u, abort_flag);
        if (!ok) break;
        mbar_expect_tx(kv_full(st), two ? L::STAGE_BYTES : L::STAGE_BYTES / 2);
        const uint32_t k_dst = kv_smem + st * L::STAGE_BYTES;
        const int pa = p_begin + 2 * j;
#pragma unroll
        for (int b = 0; b < HB; ++b) {
          const uint32_t kb = k_dst + b * (2 * L::PAGE_BOX), vb = kb + L::K_BYTES;
          load_page(pa, page_a, kb, vb, b, kv_full(st));
          if (two) load_page(pa + 1, page_b, kb + L::PAGE_BOX, vb + L::PAGE_BOX, b, kv_full(st));
        }
        if (writer && (pa + (two ? 2 : 1)) * PAGE_TOKENS > pos0 + q0) {
          // the tile's own pages are the last it reads: their stages are not filled again
          ok = mbar_wait(kv_full(st), (j / L::STAGES) & 1u, abort_flag);
          if (!ok) break;
#pragma unroll
          for (int b = 0; b < HB; ++b) {
            const uint32_t kb = k_dst + b * (2 * L::PAGE_BOX), vb = kb + L::K_BYTES;
            store_page(pa, page_a, kb, vb, b);
            if (two) store_page(pa + 1, page_b, kb + L::PAGE_BOX, vb + L::PAGE_BOX, b);
          }
          bulk_commit();
        }
      }
      if (stored) bulk_wait_all();   // the stores have left shared memory and reached the cache
      nb_launch_dependents();        // all loads are on their way: the next kernel may be set up
    }
  } else if (warp == 1) {
    if (lane == 0) {   // ------------------------------------------------------ MMA issuer
      constexpr uint32_t idesc_s2 = instr_desc_bf16(TILE_Q, 2 * PAGE_TOKENS);   // two pages of keys
      constexpr uint32_t idesc_s1 = instr_desc_bf16(TILE_Q, PAGE_TOKENS);       // one
      constexpr uint32_t idesc_o = instr_desc_bf16_b_mn(TILE_Q, HD);
      bool ok = mbar_wait(q_full, 0u, abort_flag);
      tc05_fence_after();
      // O_i = P_i V_i: A = the probabilities in tensor memory (16 keys = 8 columns per MMA),
      // B = the pages' values, MN-major: 16 keys = two groups of 8 rows, the second page 8 KB
      // after the first, the head's second 64 columns 16 KB on.  The MMAs of a CTA run in the
      // order they were issued, so the score product that later reuses this turn's score
      // buffer needs no wait of its own.
      auto value_product = [&](int i) -> bool {
        const int b = i & 1, st = i % L::STAGES;
        if (!mbar_wait(p_full(b), (i >> 1) & 1u, abort_flag)) return false;
        if (!mbar_wait(o_empty(b), ((i >> 1) & 1u) ^ 1u, abort_flag)) return false;
        tc05_fence_after();
        const uint32_t v_addr = kv_smem + st * L::STAGE_BYTES + L::K_BYTES;
        const uint32_t a_tmem = tmem_base + L::S_COL + b * (2 * PAGE_TOKENS);
        const uint32_t d_tmem = tmem_base + L::O_COL + b * HD;
        const int k_steps = two_pages(i) ? 8 : 4;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (k < k_steps) {
            const uint64_t db = smem_desc_sw128_mn(v_addr + (k >> 2) * L::PAGE_BOX + (k & 3) * 2048u,
                                                   2 * L::PAGE_BOX, 1024u);
            tc05_mma_bf16_a_tmem(d_tmem, a_tmem + k * 8, db, idesc_o, k > 0 ? 1u : 0u);
          }
        }
        tc05_commit(o_full(b));
        tc05_commit(kv_empty(st));
        return true;
      };
      for (int j = 0; j < nb && ok; ++j) {
        const int b = j & 1, st = j % L::STAGES;
        ok = mbar_wait(kv_full(st), (j / L::STAGES) & 1u, abort_flag);
        if (!ok) break;
        tc05_fence_after();
        const uint32_t k_addr = kv_smem + st * L::STAGE_BYTES;
        const uint32_t d_tmem = tmem_base + L::S_COL + b * (2 * PAGE_TOKENS);
        const uint32_t idesc_s = two_pages(j) ? idesc_s2 : idesc_s1;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          // 16 head columns per MMA: 32 bytes inside a 64-column box, the next box after four
          const uint32_t box = k >> 2, in_box = (k & 3) * 2;
          const uint64_t da = smem_desc_sw128(q_smem + box * (TILE_Q * 128)) + in_box;
          const uint64_t db = smem_desc_sw128(k_addr + box * (2 * L::PAGE_BOX)) + in_box;
          tc05_mma_bf16(d_tmem, da, db, idesc_s, k > 0 ? 1u : 0u);
        }
        tc05_commit(s_full(b));
        if (j > 0) ok = value_product(j - 1);
      }
      if (ok) value_product(nb - 1);
    }
  } else {             // ------------------------------------------------------ softmax
    // Two threads share a row: the warps 2..5 take the first page of a turn and the first
    // half of the head's columns, the warps 6..9 the second page and the second half.  The two halves of a row
    // agree on the row's maximum through shared memory once per page (a named barrier of the
    // two warps); each keeps the sum of its own keys, added up at the end.  A thread that has
    // seen a wait run out goes on through the loop without touching tensor memory, so that
    // its partner never waits for it at the barrier.
    const int quarter = warp & 3;              // the 32 tensor-memory lanes this warp may read
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;         // row of the tile
    const int qpos = pos0 + q0 + r;            // absolute position of this row's query
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const float sl2 = scale * 1.4426950408889634f;    // scores in units of log2(e)
    constexpr int OC = HD / 2;                 // output columns of this thread
    float acc[OC];
#pragma unroll
    for (int c = 0; c < OC; ++c) acc[c] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;
    float resc_prev = 0.0f;                    // rescale factor of the page before
    bool ok = true;
    auto pair_barrier = [&]() {   // the two warps of a quarter; barrier numbers 1..4
      switch (quarter) {
        case 0: asm volatile("bar.sync 1, 64;\n" ::: "memory"); break;
        case 1: asm volatile("bar.sync 2, 64;\n" ::: "memory"); break;
        case 2: asm volatile("bar.sync 3, 64;\n" ::: "memory"); break;
        default: asm volatile("bar.sync 4, 64;\n" ::: "memory"); break;
      }
    };
    // one lane polls for the warp
    auto warp_wait = [&](uint32_t bar, uint32_t parity) -> bool {
      int got = 1;
      if (lane == 0) got = (int)mbar_wait(bar, parity, abort_flag);
      return __shfl_sync(0xffffffffu, got, 0) != 0;
    };
    // acc = acc * resc + O_i, with this thread's columns of O_i read from tensor memory
    auto take_output = [&](int i, float resc) -> bool {
      const int b = i & 1;
      if (!warp_wait(o_full(b), (i >> 1) & 1u)) return false;
      tc05_fence_after();
#pragma unroll
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t ov[32];
        tc05_ld_32x32b_x32(lane_addr + L::O_COL + b * HD + half * OC + c * 32, ov);
        tc05_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) acc[c * 32 + e] = fmaf(acc[c * 32 + e], resc, __uint_as_float(ov[e]));
      }
      tc05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_empty(b));
      return true;
    };

    for (int j = 0; j < nb; ++j) {
      const int b = j & 1;
      const bool has_keys = half == 0 || two_pages(j);   // a turn may have one page only
      uint32_t v0[32], v1[32];
      if (ok) ok = warp_wait(s_full(b), (j >> 1) & 1u);
      if (ok && has_keys) {
        tc05_fence_after();
        tc05_ld_32x32b_x32(lane_addr + L::S_COL + b * (2 * PAGE_TOKENS) + half * PAGE_TOKENS, v0);
        tc05_ld_32x32b_x32(lane_addr + L::S_COL + b * (2 * PAGE_TOKENS) + half * PAGE_TOKENS + 32, v1);
        tc05_wait_ld();
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) v0[e] = v1[e] = 0u;
      }

      // causal limit and window; the maximum of this thread's 64 keys.  A turn that lies
      // wholly before the first row of this warp (and needs no window) is visible to all of
      // its rows.  Bit e of `vis`: key k0 + e counts for this row.
      const int k0 = (p_begin + 2 * j + half) * PAGE_TOKENS;
      const bool all_visible =
          window <= 0 && two_pages(j) &&
          (p_begin + 2 * j + 2) * PAGE_TOKENS - 1 <= pos0 + q0 + quarter * 32;
      unsigned long long vis = 0ull;
      if (has_keys) {
        const int hi = qpos - k0;                                   // keys 0..hi are not in the future
        const int lo = window > 0 ? qpos - window + 1 - k0 : 0;     // keys lo.. are inside the window
        const unsigned long long up = hi >= 63 ? ~0ull : (hi < 0 ? 0ull : ((2ull << hi) - 1ull));
        const unsigned long long dn = lo <= 0 ? ~0ull : (lo > 63 ? 0ull : (~0ull << lo));
        vis = up & dn;
      }
      // The scale is positive (the launcher sees to it), so the maximum is taken over the raw
      // scores and scaled once, and the scaling of a score is folded into its exponent.
      float x[64];
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (all_visible) {
#pragma unroll
        for (int e = 0; e < 64; ++e) {
          x[e] = __uint_as_float(e < 32 ? v0[e] : v1[e - 32]);
          mx4[e & 3] = fmaxf(mx4[e & 3], x[e]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 64; ++e) {
          x[e] = ((vis >> e) & 1ull) ? __uint_as_float(e < 32 ? v0[e] : v1[e - 32]) : -INFINITY;
          mx4[e & 3] = fmaxf(mx4[e & 3], x[e]);
        }
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sl2;
      xch[(b * 2 + half) * TILE_Q + r] = mx;
      pair_barrier();   // also: both halves have read their scores, which the probabilities overwrite
      mx = fmaxf(mx, xch[(b * 2 + (half ^ 1)) * TILE_Q + r]);
      const float m_new = fmaxf(m_run, mx);
      const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
      const float resc = (m_run == -INFINITY) ? 0.0f : nb_exp2(m_run - m_use);
      m_run = m_new;
      float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      uint32_t pk[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const float p0 = nb_exp2(fmaf(x[2 * e], sl2, -m_use));
        const float p1 = nb_exp2(fmaf(x[2 * e + 1], sl2, -m_use));
        sum4[e & 3] += p0 + p1;
        const __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
        pk[e] = *reinterpret_cast<const uint32_t*>(&hh);
      }
      l_run = fmaf(l_run, resc, (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));

      // this thread's probabilities: 64 bf16 = 32 columns of the row, over the scores
      if (ok) {
        if (has_keys) {
          tc05_st_32x32b_x32(lane_addr + L::S_COL + b * (2 * PAGE_TOKENS) + half * 32, pk);
          tc05_wait_st();
        }
        if (j == nb - 1 && p_end == p_last && tail_row < PAGE_TOKENS) {
          // Rows of the sequence's last page after its newest key hold whatever an earlier
          // owner of the page left there (or, read from the step's rows, a neighbour's keys).
          // Their probabilities are zero, but zero times a non-finite value is not: the eight
          // softmax warps clear those value rows in the staged page before the value product
          // may start (it waits for all of them at p_full).  A row is 128 bytes inside each
          // 64-column box, whatever the swizzle does within it.
          unsigned char* vpage = gen + L::Q_BYTES + (j % L::STAGES) * L::STAGE_BYTES + L::K_BYTES +
                                 ((p_end - 1) - (p_begin + 2 * j)) * L::PAGE_BOX;
          const int sm_tid = (warp - 2) * 32 + lane;
          for (int i = sm_tid; i < (PAGE_TOKENS - tail_row) * 8 * HB; i += 256) {
            const int box = i / ((PAGE_TOKENS - tail_row) * 8), rem = i % ((PAGE_TOKENS - tail_row) * 8);
            *reinterpret_cast<uint4*>(vpage + box * (2 * L::PAGE_BOX) + (tail_row + rem / 8) * 128 +
                                      (rem % 8) * 16) = make_uint4(0u, 0u, 0u, 0u);
          }
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        }
        tc05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full(b));
        if (j > 0) ok = take_output(j - 1, resc_prev);
      }
      resc_prev = resc;
    }
    if (ok) ok = take_output(nb - 1, resc_prev);

    // the row's sum: both halves
    xch[(4 + half) * TILE_Q + r] = l_run;
    pair_barrier();
    l_run += xch[(4 + (half ^ 1)) * TILE_Q + r];

    bool write_out = ok;
    if (n_splits > 1) {
      // partial result of this run of pages: per row the maximum and the sum, then the
      // unnormalised outputs; all in units of this CTA's own maximum
      constexpr int REC = 2 * TILE_Q + TILE_Q * HD;          // floats per (tile, split)
      const size_t tile_id = ((size_t)s * gridDim.y + h) * (gridDim.x / max_splits) + tile;
      float* mine = part + (tile_id * max_splits + split) * REC;
      if (ok) {
        if (half == 0) {
          mine[r] = m_run;
          mine[TILE_Q + r] = l_run;
        }
        float* po = mine + 2 * TILE_Q + (size_t)r * HD + half * OC;
#pragma unroll
        for (int c = 0; c < OC / 4; ++c)
          *reinterpret_cast<float4*>(po + c * 4) =
              make_float4(acc[c * 4], acc[c * 4 + 1], acc[c * 4 + 2], acc[c * 4 + 3]);
      }
      __threadfence();
      asm volatile("bar.sync 5, 256;\n" ::: "memory");     // the eight softmax warps
      if (warp == 2 && lane == 0) {
        const int old = atomicAdd(&counters[tile_id], 1);
        const int last = (old == n_splits - 1);
        if (last) counters[tile_id] = 0;                    // ready for the next launch
        xch[0] = last ? 1.0f : 0.0f;
      }
      asm volatile("bar.sync 5, 256;\n" ::: "memory");
      write_out = ok && xch[0] != 0.0f;
      if (write_out) {
        __threadfence();
        const float* all = part + tile_id * max_splits * REC;
        float m_all = -INFINITY;
        for (int i = 0; i < n_splits; ++i) m_all = fmaxf(m_all, __ldcg(all + (size_t)i * REC + r));
        const float m_ref = (m_all == -INFINITY) ? 0.0f : m_all;
        l_run = 0.0f;
#pragma unroll
        for (int c = 0; c < OC; ++c) acc[c] = 0.0f;
        for (int i = 0; i < n_splits; ++i) {                // in the order of the pages
          const float* rec = all + (size_t)i * REC;
          const float m_i = __ldcg(rec + r);
          const float w = (m_i == -INFINITY) ? 0.0f : nb_exp2(m_i - m_ref);
          l_run = fmaf(__ldcg(rec + TILE_Q + r), w, l_run);
          const float* po = rec + 2 * TILE_Q + (size_t)r * HD + half * OC;
#pragma unroll
          for (int c = 0; c < OC / 4; ++c) {
            const float4 f = __ldcg(reinterpret_cast<const float4*>(po + c * 4));
            acc[c * 4] = fmaf(f.x, w, acc[c * 4]);
            acc[c * 4 + 1] = fmaf(f.y, w, acc[c * 4 + 1]);
            acc[c * 4 + 2] = fmaf(f.z, w, acc[c * 4 + 2]);
            acc[c * 4 + 3] = fmaf(f.w, w, acc[c * 4 + 3]);
          }
        }
      }
    }

    if (write_out && r < rows_here) {
      const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
      TOut* dst = out + (size_t)(row0 + q0 + r) * out_stride + (size_t)h * HD + half * OC;
      if constexpr (sizeof(TOut) == 2) {
#pragma unroll
        for (int c = 0; c < OC / 8; ++c) {
          uint4 u;
          __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
          for (int e = 0; e < 4; ++e)
            hh[e] = __floats2bfloat162_rn(acc[c * 8 + 2 * e] * inv, acc[c * 8 + 2 * e + 1] * inv);
          *reinterpret_cast<uint4*>(dst + c * 8) = u;
        }
      } else {
#pragma unroll
        for (int c = 0; c < OC / 4; ++c)
          *reinterpret_cast<float4*>(dst + c * 4) =
              make_float4(acc[c * 4] * inv, acc[c * 4 + 1] * inv, acc[c * 4 + 2] * inv,
                          acc[c * 4 + 3] * inv);
      }
    }
  }

  tc05_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) {
      nb_report_timeout(err_word);
      // let TMA copies that are still in flight land before the shared memory goes away
      const long long t0 = clock64();
      while (clock64() - t0 < 4000000LL) {
      }
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base),
                 "r"((uint32_t)L::TMEM_COLS)
                 : "memory");
  }
}

// The word of pinned host memory in which this kernel reports a wait that ran out.
int* error_word() {
  int* w = nb_error_words();
  return w ? w + NB_ERRW_ATTENTION_PREFILL_TC : nullptr;
}

template <int HD, typename TOut>
int launch_tc(const void* q, int q_stride, int q_col, int n_rows, const int* cu_rows,
              const int* seq_slot, const int* seq_pos0, const void* k_cache, const void* v_cache,
              long long n_pages, const int* block_table, int max_pages, int n_heads, int n_kv_heads,
              void* out, int out_stride, float scale, int window, int n_seqs, int max_q_len,
              int max_splits, int chunk_pages, float* part, int* counters, int append, int k_col,
              int v_col, cudaStream_t stream) {
  using L = AttnSmem<HD>;
  CUtensorMap mq, mk, mv, mn;
  int rc = make_map(&mq, q, n_rows, q_stride, TILE_Q, 64, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2);
  if (rc) return rc;
  const long long kv_rows = n_pages * n_kv_heads * PAGE_TOKENS;
  rc = make_map(&mk, k_cache, kv_rows, HD, PAGE_TOKENS, 64, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2);
  if (rc) return rc;
  rc = make_map(&mv, v_cache, kv_rows, HD, PAGE_TOKENS, 64, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2);
  if (rc) return rc;
  rc = make_map(&mn, q, n_rows, q_stride, PAGE_TOKENS, 64, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2);
  if (rc) return rc;
  auto kern = attention_prefill_tc_kernel<HD, TOut>;
  static bool configured = false;   // per instantiation
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    configured = true;
  }
  dim3 grid(((max_q_len + TILE_Q - 1) / TILE_Q) * max_splits, n_heads, n_seqs);
  NB_CUDA(nb_launch(kern, grid, dim3(TC_THREADS), (size_t)L::TOTAL, stream, mq, mk, mv, mn, append, k_col,
                    v_col, q_col, cu_rows, seq_slot, seq_pos0, block_table, max_pages, n_kv_heads,
                    n_heads / n_kv_heads, (TOut*)out, out_stride, scale, window, max_splits,
                    chunk_pages, part, counters, error_word()));
  return 0;
}

}  // namespace

// 1 if the tensor-core prefill kernel takes this shape.
NB_EXPORT int nb_attention_prefill_tc_supported(int dtype, int head_dim, int n_heads,
                                                int n_kv_heads, int page, int q_stride, int q_col,
                                                int out_dtype, int out_stride) {
  if (dtype != NB_BF16 || page != PAGE_TOKENS) return 0;
  if (n_kv_heads < 1 || n_heads % n_kv_heads != 0) return 0;
  if (q_stride % 8 != 0 || q_col % 8 != 0) return 0;            // TMA: 16-byte pitch and start
  if (out_stride % (out_dtype == NB_F32 ? 4 : 8) != 0) return 0;  // 16-byte output stores
  return head_dim == 64 || head_dim == 128;
}

// Waits for the device, then reads (and lowers) the word that a timed-out wait of this kernel
// raises.
NB_EXPORT int nb_attention_prefill_tc_error() {
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  volatile int* w = error_word();
  if (w == nullptr) return 0;
  const int v = *w;
  if (v) *w = 0;
  return v;
}

// Clock cycles a wait of this kernel may take before it gives up (default 4e9).
NB_EXPORT int nb_attention_prefill_tc_set_wait_budget(long long cycles) {
  NB_REQUIRE(cycles >= 0, NB_ERR_BAD_ARG, "wait budget must not be negative");
  return set_wait_budget(cycles);
}

// Floats of scratch per (sequence, head, 128-row tile, split) when the pages of a tile are cut
// into more than one run.
NB_EXPORT int nb_attention_prefill_tc_record(int head_dim) { return 2 * TILE_Q + TILE_Q * head_dim; }

// Rows of sequence s are cu_rows[s]..cu_rows[s+1] of the packed batch (n_rows rows of q_stride
// elements), at positions seq_pos0[s].. of slot seq_slot[s]; their keys and values are already
// in the cache, which holds n_pages pages.  max_splits > 1 cuts the pages a tile reads into
// runs of chunk_pages (max_splits * chunk_pages must cover the longest sequence); it needs
// `part` (n_seqs * n_heads * tiles * max_splits records) and `counters` (one int per
// (sequence, head, tile), zero before the first use; every launch leaves them at zero).
// append != 0: the rows also hold the step's keys and values at columns k_col / v_col (key/value
// head after head); every seq_pos0 must then be a multiple of the page size, and the kernel
// writes them to the cache itself.
NB_EXPORT int nb_attention_prefill_tc(const void* q, int dtype, int q_stride, int q_col, int n_rows,
                                      const int* cu_rows, const int* seq_slot, const int* seq_pos0,
                                      const void* k_cache, const void* v_cache, int n_pages,
                                      const int* block_table, int max_pages, int page, int n_heads,
                                      int n_kv_heads, int head_dim, void* out, int out_dtype,
                                      int out_stride, float scale, int window, int n_seqs,
                                      int max_q_len, int max_splits, int chunk_pages, float* part,
                                      int* counters, int append, int k_col, int v_col,
                                      cudaStream_t stream) {
  if (n_seqs == 0 || max_q_len == 0) return 0;
  NB_REQUIRE(nb_attention_prefill_tc_supported(dtype, head_dim, n_heads, n_kv_heads, page, q_stride,
                                               q_col, out_dtype, out_stride),
             NB_ERR_UNSUPPORTED,
             "attention_prefill_tc: unsupported shape (head size %d, %d/%d heads, row pitch %d)",
             head_dim, n_heads, n_kv_heads, q_stride);
  NB_REQUIRE(n_seqs <= 65535 && n_heads <= 65535 && n_rows > 0 && n_pages > 0, NB_ERR_UNSUPPORTED,
             "attention_prefill_tc: bad sizes");
  NB_REQUIRE(!append || (k_col % 8 == 0 && v_col % 8 == 0 && k_col >= 0 && v_col >= 0),
             NB_ERR_UNSUPPORTED, "attention_prefill_tc: key/value columns %d/%d are not 16-byte aligned",
             k_col, v_col);
  NB_REQUIRE(scale > 0.0f, NB_ERR_UNSUPPORTED, "attention_prefill_tc: takes a positive scale (got %g)",
             (double)scale);
  NB_REQUIRE(max_splits >= 1 && chunk_pages >= 1 && (max_splits == 1 || (part && counters)) &&
                 (uintptr_t)part % 16 == 0,
             NB_ERR_BAD_ARG, "attention_prefill_tc: bad split (%d runs of %d pages)", max_splits,
             chunk_pages);
  NB_REQUIRE((long long)((max_q_len + TILE_Q - 1) / TILE_Q) * max_splits <= 2147483647LL,
             NB_ERR_UNSUPPORTED, "attention_prefill_tc: grid too large");
  NB_REQUIRE((uintptr_t)q % 16 == 0 && (uintptr_t)k_cache % 16 == 0 && (uintptr_t)v_cache % 16 == 0 &&
                 (uintptr_t)out % 16 == 0,
             NB_ERR_UNSUPPORTED, "attention_prefill_tc: operands must be 16-byte aligned");
  int rc = NB_ERR_UNSUPPORTED;
#define NB_ARGS q, q_stride, q_col, n_rows, cu_rows, seq_slot, seq_pos0, k_cache, v_cache, (long long)n_pages, block_table, max_pages, n_heads, n_kv_heads, out, out_stride, scale, window, n_seqs, max_q_len, max_splits, chunk_pages, part, counters, append, k_col, v_col, stream
  if (head_dim == 64)
    rc = out_dtype == NB_F32 ? launch_tc<64, float>(NB_ARGS) : launch_tc<64, bf16>(NB_ARGS);
  else
    rc = out_dtype == NB_F32 ? launch_tc<128, float>(NB_ARGS) : launch_tc<128, bf16>(NB_ARGS);
#undef NB_ARGS
  if (rc) return rc;
  NB_CHECK_LAUNCH("attention_prefill_tc");
  return 0;
}
