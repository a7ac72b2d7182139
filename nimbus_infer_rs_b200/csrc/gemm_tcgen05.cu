// Matrix product on the 5th-generation tensor cores (sm_100a): out[M,N] = act(X[M,K] *
// W[N,K]^T + bias) (+ residual), bf16 operands, fp32 accumulation in tensor memory.
//
// A CTA computes 128 x BN tiles (BN = 64, 96, 128, 192 or 256, picked so that the tiles fill
// the SMs in as few waves as possible), one after another.  Warp 0 is the producer: one thread issues TMA loads of
// 128 x 64 (X) and BN x 64 (W) bf16 boxes, 128-byte swizzled, into a ring of shared-memory
// stages, each guarded by a full/empty mbarrier pair.  Warp 1 owns the tensor memory
// allocation and one of its threads issues `tcgen05.mma` (M=128, N=BN, K=16; four per stage)
// with shared-memory matrix descriptors; `tcgen05.commit` hands a stage back to the producer
// and, after the last K block of a tile, signals that tile's accumulator (there are two, used
// in turn).  The other 8 or 16 warps are the epilogue: each reads its share of the columns of
// its 32-lane quarter of the accumulator with `tcgen05.ld`, hands the accumulator back, applies bias / GELU / residual in fp32 and
// stores its rows while the MMAs of the next tile already run.  Edges need no special code on the load side: TMA
// zero-fills rows beyond M or N and columns beyond K.
//
// Every wait on an mbarrier is bounded by a clock budget; a wait that runs out raises an
// error flag (nb_gemm_tcgen05_error), all roles leave their loops, the CTA lets its copies in
// flight land, frees its tensor memory and returns.
//
// Requirements: K % 8 == 0 (16-byte row pitch for TMA), 16-byte aligned bases.
// Reference analogue: Mat::gemm_into (src/model.rs:94-133).
#include "tc05_common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

// Tuning (nb_gemm_tcgen05_tune): whether a CTA with one tile and a long K has two MMA-issuing
// threads, and whether the producer is more than one lane.  What a launch passes to the
// kernel: bit 0: two issuing threads; bits 1-2: the producer is 0 one lane, 1 a lane for X and
// a lane for W (large tiles), 2 lanes that share out the ring's stages (a single row tile).
bool g_dual = true, g_lanes = true;

constexpr int BM = 128;
constexpr int BK = 64;               // 64 bf16 = 128 bytes = one swizzle atom row
constexpr int UMMA_K = 16;
// Epilogue warps per CTA: a warp may read only the 32 tensor-memory lanes of its quarter
// (warp index mod 4), so the warps of a quarter share the tile's columns among them.
// With the direct-store epilogue (EPI 0) there are 16 warps for wide tiles, 8 otherwise; with
// the shared-memory / TMA-store epilogue (EPI 1) every warp owns 64 columns of its quarter.
__host__ __device__ constexpr int epi_warps(int bn, int epi) {
  return epi ? 4 * ((bn + 63) / 64) : (bn >= 128 ? 16 : 8);
}
// Tensor-memory columns between the two accumulators of a CTA: allocations are powers of two.
__host__ __device__ constexpr int acc_stride(int bn) {
  return bn <= 64 ? 64 : (bn <= 128 ? 128 : 256);
}
__host__ __device__ constexpr int cta_threads(int bn, int epi) { return 64 + 32 * epi_warps(bn, epi); }

// One CTA per SM walks over tiles; two accumulators in tensor memory let the epilogue of one
// tile overlap the main loop of the next.  EPI 1 adds a staging area for the epilogue: 4 KB
// (32 rows x 128 bytes, 128-byte swizzled) per epilogue warp for bf16 output, twice that for
// fp32 output (two 32-column boxes per warp, which also receive the residual by TMA).
// PAIR 1: two CTAs of a cluster share 256 x BN tiles (`cta_group::2`): each brings its 128
// rows of X and half of the tile's rows of W, so a stage holds BN / 2 rows of W.
template <int BN, int EPI, int ESIZE, int PAIR>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_WARPS = epi_warps(BN, EPI);
  static constexpr int STG_PER_WARP = EPI ? (ESIZE == 4 ? 8192 : 4096) : 0;
  static constexpr int STG_BYTES = EPI_WARPS * STG_PER_WARP;
  static constexpr int BUDGET = 222 * 1024;   // of the 227 KB a CTA may have
  static constexpr int STAGES_RAW = (BUDGET - STG_BYTES) / STAGE_BYTES;
  // 2, 3, 4, 6 or 8 stages: the producer lanes share the stages out among them (see the kernel)
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : (STAGES_RAW == 7 ? 6 : (STAGES_RAW == 5 ? 4 : STAGES_RAW));
  static constexpr int PRODUCERS = PAIR ? 1 : (STAGES % 4 == 0 ? 4 : (STAGES % 3 == 0 ? 3 : (STAGES % 2 == 0 ? 2 : 1)));
  static constexpr int TILES_BYTES = STAGES * STAGE_BYTES;
  // after tiles and staging: full[STAGES], empty[STAGES], accumulator full[2] / empty[2], two
  // residual barriers per epilogue warp, then the tensor-memory base address and the abort flag
  static constexpr int N_BARRIERS = 2 * STAGES + 4 + 2 * EPI_WARPS;
  static constexpr int TOTAL = TILES_BYTES + STG_BYTES + N_BARRIERS * 8 + 16 + 1024 /* alignment slack */;
};

template <int BN, int EPI, typename TOut, int PAIR>
__global__ void __launch_bounds__(cta_threads(BN, EPI))
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_out, const float* __restrict__ bias,
                    const float* residual, TOut* out, int M, int N, int K, int act, int tiles_n,
                    int num_tiles, int a_box_bytes, int* err_word, int tune) {
  using L = SmemLayout<BN, EPI, (int)sizeof(TOut), PAIR>;
  constexpr int EW = L::EPI_WARPS;
  constexpr int ACC = acc_stride(BN);
  static_assert(!PAIR || (EPI == 1 && BN % 32 == 0), "paired CTAs: TMA epilogue only");
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "tile width");
  static_assert(EPI == 1 || BN == 64 || BN == 128 || BN == 256, "direct-store epilogue: 64/128/256");
  static_assert(BN % 64 == 0 || (EPI == 1 && sizeof(TOut) == 4), "odd widths: fp32 TMA epilogue only");
  extern __shared__ unsigned char smem_dyn[];
  // 1024-byte alignment (swizzle atoms), computed on the shared-window address
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* gen = smem_dyn + (base - raw);
  const uint32_t stg_base = base + L::TILES_BYTES;          // epilogue staging (EPI 1)
  const uint32_t bars = stg_base + L::STG_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (L::STAGES + s); };
  auto acc_full = [&](int b) { return bars + 8u * (2 * L::STAGES + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (2 * L::STAGES + 2 + b); };
  auto res_bar = [&](int w, int u) { return bars + 8u * (2 * L::STAGES + 4 + 2 * w + u); };
  uint32_t* tmem_slot =
      reinterpret_cast<uint32_t*>(gen + L::TILES_BYTES + L::STG_BYTES + L::N_BARRIERS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int num_kb = (K + BK - 1) / BK;
  // Paired CTAs: rank 0 is the leader.  It alone issues the MMAs (which read both CTAs'
  // shared memory and write both CTAs' tensor memory); the TMA loads of both CTAs count on the
  // leader's full barriers; commits go to the barriers of both; the epilogue warps of both tell
  // the leader's accumulator-empty barriers.
  uint32_t rank = 0;
  if constexpr (PAIR) asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
  const int walker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;    // who walks over tiles
  const int n_walkers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int m_off = PAIR ? (int)rank * BM : 0;                   // this CTA's rows in a tile
  constexpr int TILE_M = PAIR ? 2 * BM : BM;

  if (tid == 0) {
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
    if constexpr (EPI == 1) prefetch_tensormap(&map_out);
    for (int s = 0; s < L::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), PAIR ? 2 * EW : EW);   // one arrival per epilogue warp (of both CTAs)
    }
    for (int w = 0; w < EW; ++w) {
      mbar_init(res_bar(w, 0), 1);
      mbar_init(res_bar(w, 1), 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if constexpr (PAIR) {   // the peer's barriers exist before anything of ours can reach them
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
  }
  if (warp == 1) {   // the whole warp allocates two accumulators, ACC columns apart
    if constexpr (PAIR) {   // warp 1 of both CTAs, the same columns in both
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                       smem_u32(tmem_slot)),
                   "r"((uint32_t)(2 * ACC))
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                       smem_u32(tmem_slot)),
                   "r"((uint32_t)(2 * ACC))
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
  }
  tc05_fence_before();
  __syncthreads();
  tc05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Barriers and tensor memory are set up; what the kernel before this one wrote (the rows of
  // X, the residual) is touched from here on.  Under a programmatic launch the set-up above
  // ran while that kernel was finishing -- and so do the loads of the first tile's weights
  // (constants): a product of a decode step is a few microseconds long, and the trip to HBM
  // for its first weights would be a good part of that.
  int pre_kb = 0;   // K blocks whose weights are already on their way (the producer's)
  if constexpr (!PAIR) {
    if (tid == 0 && walker < num_tiles) {
      pre_kb = num_kb < L::STAGES ? num_kb : L::STAGES;
      const int n0 = (walker % tiles_n) * BN;
      for (int kb = 0; kb < pre_kb; ++kb) {
        mbar_expect_tx(full_bar(kb), (uint32_t)a_box_bytes + L::B_BYTES);
        tma_load_2d(base + kb * L::STAGE_BYTES + L::A_BYTES, &map_w, kb * BK, n0, full_bar(kb));
      }
    }
  }
  nb_grid_dependency_wait();
  if (warp == 0) pre_kb = __shfl_sync(0xffffffffu, pre_kb, 0);   // the producer lanes all need it

  // Two issuing threads.  A `tcgen05.mma` costs the thread that issues it about 80 clocks
  // whatever its width, so a CTA with one tile and a long K (a decode step, a short prompt) is
  // bound by that thread while the tensor cores idle; two threads with an accumulator each
  // get rid of an instruction every 50 clocks between them.  The first takes the even blocks
  // of K into the first accumulator, lane 0 of the first epilogue warp (idle until then) the
  // odd ones into the second, and the epilogue adds the two.
  const bool dual = !PAIR && (tune & 1) && num_tiles <= n_walkers && num_kb >= 8;
  auto dual_walk = [&](int first) {
    constexpr uint32_t idesc = instr_desc_bf16(TILE_M, BN);
    const uint32_t d_tmem = tmem_base + (uint32_t)first * ACC;
    bool ok = walker < num_tiles;
    for (int kb = first; kb < num_kb && ok; kb += 2) {
      const int s = kb % L::STAGES;
      ok = mbar_wait(full_bar(s), (uint32_t)(kb / L::STAGES) & 1u, abort_flag);
      if (!ok) break;
      tc05_fence_after();
      const uint32_t a_addr = base + s * L::STAGE_BYTES;
      const uint64_t da = smem_desc_sw128(a_addr);
      const uint64_t db = smem_desc_sw128(a_addr + L::A_BYTES);
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k)
        tc05_mma_bf16(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                      (kb > first || k > 0) ? 1u : 0u);
      tc05_commit(empty_bar(s));
    }
    if (ok) tc05_commit(acc_full(first));
  };

  // The CTA walks over output tiles blockIdx.x, blockIdx.x + gridDim.x, ...; the shared-memory
  // ring runs on across tiles, and while the epilogue drains one accumulator the MMAs of the
  // next tile fill the other.
  //
  // A TMA tile load costs its issuing thread about 190 clocks whatever the size of the box
  // (measured: 16 to 256 rows of 128 bytes), so one thread brings in at most 85 bytes a clock
  // with the two boxes of a wide tile and 40 with those of a 64-row product; four lanes of the
  // producer's warp, each with every fourth block of K, reach what the TMA unit takes (about
  // 100 bytes a clock).
  // The number of lanes divides the number of stages, so a lane owns its stages: it fills a
  // stage again only after its own earlier wait for that stage, and can never be two rounds
  // of the ring ahead of the MMAs that free it (where the parity of an older phase of the
  // stage's barrier would pass for the one it waits for), in whatever order two issuing
  // threads consume the stages.
  const int PRODUCERS = (tune >> 1) == 2 ? L::PRODUCERS : 1;
  // Large tiles: one lane brings
  // the rows of X, the other the rows of W, both block after block in order, so the ring
  // fills in the order the MMAs read it at twice one thread's issue rate.  The lane of X arms
  // the stage's barrier with the bytes of both boxes; bytes of W that land before that only
  // take the count below zero for a while (the phase cannot end before the arming arrives).
  const bool split_xw = !PAIR && (tune >> 1) == 1;
  if (warp == 0 && split_xw) {
    if (lane < 2) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = walker; tile < num_tiles && ok; tile += n_walkers) {
        const int m0 = (tile / tiles_n) * TILE_M + m_off;
        const int n0 = (tile % tiles_n) * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % L::STAGES;
          const uint32_t phase = (it / L::STAGES) & 1u;
          const bool early = tile == walker && kb < pre_kb;   // armed, W on its way since before the wait
          if (!early) ok = mbar_wait(empty_bar(s), phase ^ 1u, abort_flag);
          if (!ok) break;
          const uint32_t a_dst = base + s * L::STAGE_BYTES;
          if (lane == 0) {
            if (!early) mbar_expect_tx(full_bar(s), (uint32_t)a_box_bytes + L::B_BYTES);
            tma_load_2d(a_dst, &map_x, kb * BK, m0, full_bar(s));
          } else if (!early) {
            tma_load_2d(a_dst + L::A_BYTES, &map_w, kb * BK, n0, full_bar(s));
          }
        }
      }
      nb_launch_dependents();
    }
  } else if (warp == 0) {
    if (lane < PRODUCERS) {   // --------------------------------------------- TMA producers
      uint32_t it_tile = 0;
      bool ok = true;
      for (int tile = walker; tile < num_tiles && ok; tile += n_walkers, it_tile += (uint32_t)num_kb) {
        const int m0 = (tile / tiles_n) * TILE_M + m_off;
        const int n0 = (tile % tiles_n) * BN + (PAIR ? (int)rank * (BN / 2) : 0);
        // a lane takes every PRODUCERS-th block of the CTA's whole walk (across its tiles)
        const int kb_first = (int)(((uint32_t)lane + PRODUCERS - it_tile % PRODUCERS) % PRODUCERS);
        for (int kb = kb_first; kb < num_kb; kb += PRODUCERS) {
          const uint32_t it = it_tile + (uint32_t)kb;
          const int s = it % L::STAGES;
          const uint32_t phase = (it / L::STAGES) & 1u;
          if (!(tile == walker && kb < pre_kb)) ok = mbar_wait(empty_bar(s), phase ^ 1u, abort_flag);
          if (!ok) break;
          const uint32_t a_dst = base + s * L::STAGE_BYTES;
          if constexpr (PAIR) {
            // both CTAs' bytes are counted on the leader's barrier, which the leader arms
            if (rank == 0) mbar_expect_tx(full_bar(s), 2u * ((uint32_t)a_box_bytes + L::B_BYTES));
            const uint32_t lead_bar = cluster_addr(full_bar(s), 0);
            tma_load_2d_pair(a_dst, &map_x, kb * BK, m0, lead_bar);
            tma_load_2d_pair(a_dst + L::A_BYTES, &map_w, kb * BK, n0, lead_bar);
          } else if (tile == walker && kb < pre_kb) {
            // the stage was armed and its weights asked for before the wait: the rows follow
            tma_load_2d(a_dst, &map_x, kb * BK, m0, full_bar(s));
          } else {
            // the X box has fewer than 128 rows when the whole product has (see the launcher)
            mbar_expect_tx(full_bar(s), (uint32_t)a_box_bytes + L::B_BYTES);
            tma_load_2d(a_dst, &map_x, kb * BK, m0, full_bar(s));
            tma_load_2d(a_dst + L::A_BYTES, &map_w, kb * BK, n0, full_bar(s));
          }
        }
      }
      // every load of this CTA is on its way: the next kernel may be set up while the last
      // products and the epilogue run
      nb_launch_dependents();
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0 && dual) {
      dual_walk(0);
    } else if (lane == 0 && rank == 0) {   // ----------------------------------- MMA issuer
      constexpr uint32_t idesc = instr_desc_bf16(TILE_M, BN);
      uint32_t it = 0, t = 0;
      bool ok = true;
      for (int tile = walker; tile < num_tiles && ok; tile += n_walkers, ++t) {
        const uint32_t ab = t & 1u, aphase = (t >> 1) & 1u;
        ok = mbar_wait(acc_empty(ab), aphase ^ 1u, abort_flag);   // the epilogue has drained it
        if (!ok) break;
        tc05_fence_after();
        const uint32_t d_tmem = tmem_base + ab * ACC;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % L::STAGES;
          const uint32_t phase = (it / L::STAGES) & 1u;
          ok = mbar_wait(full_bar(s), phase, abort_flag);
          if (!ok) break;
          tc05_fence_after();
          const uint32_t a_addr = base + s * L::STAGE_BYTES;
          const uint64_t da = smem_desc_sw128(a_addr);
          const uint64_t db = smem_desc_sw128(a_addr + L::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing K by 16 elements inside the swizzle atom = 32 bytes = 2 address units
            if constexpr (PAIR)
              tc05_mma_bf16_pair(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                                 (kb > 0 || k > 0) ? 1u : 0u);
            else
              tc05_mma_bf16(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                            (kb > 0 || k > 0) ? 1u : 0u);
          }
          // the stage is free (in both CTAs) once these MMAs have read it
          if constexpr (PAIR) tc05_commit_pair(empty_bar(s)); else tc05_commit(empty_bar(s));
        }
        // complete once all MMAs issued so far are done
        if (ok) { if constexpr (PAIR) tc05_commit_pair(acc_full(ab)); else tc05_commit(acc_full(ab)); }
      }
    }
  } else if constexpr (EPI == 1) {   // ---------- epilogue through shared memory and TMA stores
    // Warp e of the epilogue owns the 32 tensor-memory lanes of its quarter and one 64-column
    // unit of the tile (the last unit of a 96-wide tile has 32).  bf16 output: the unit is one
    // 32 x 64 box; fp32 output: 32 x 32 boxes, each in a buffer of its own, into which the
    // residual (the output tensor itself, updated in place) is brought by TMA while the
    // accumulator is still being computed.  Rows and columns beyond M and N are clipped by the
    // TMA unit.
    constexpr bool F32 = sizeof(TOut) == 4;
    const int e = warp - 2;
    const int quarter = warp & 3;
    const int unit = e >> 2;                     // 64 columns each
    const int nch = (unit * 64 + 64 <= BN) ? 2 : 1;   // 32-column chunks of this warp's unit
    const uint32_t stg = stg_base + (uint32_t)e * L::STG_PER_WARP;
    const uint32_t my_row = stg + (uint32_t)lane * 128u;
    const uint32_t swz = (uint32_t)(lane & 7);
    uint32_t t = 0;
    const uint32_t lead_empty0 = PAIR ? cluster_addr(acc_empty(0), 0) : 0u;
    if (dual) {   // the second issuing thread, before its warp turns to the epilogue
      if (e == 0 && lane == 0) dual_walk(1);
      __syncwarp();
    }
    for (int tile = walker; tile < num_tiles; tile += n_walkers, ++t) {
      const int m0 = (tile / tiles_n) * TILE_M + m_off, n0 = (tile % tiles_n) * BN;
      const int row0 = m0 + quarter * 32, col0 = n0 + unit * 64;
      const uint32_t ab = t & 1u, aphase = (t >> 1) & 1u;
      if (lane == 0) {
        bulk_wait_read_all();   // the stores of the previous tile have read this warp's buffers
        if (F32 && residual != nullptr) {
          for (int u = 0; u < nch; ++u) {
            mbar_expect_tx(res_bar(e, u), 4096u);
            tma_load_2d(stg + u * 4096u, &map_out, col0 + u * 32, row0, res_bar(e, u));
          }
        }
      }
      __syncwarp();
      // the bias of this warp's columns (a constant) is fetched while the products still run:
      // behind the accumulator it would be a trip to memory at the very end of the kernel
      float bias_pre[2] = {0.0f, 0.0f};
#pragma unroll
      for (int c = 0; c < 2; ++c)
        if (bias && c < nch && col0 + c * 32 + lane < N) bias_pre[c] = __ldg(bias + col0 + c * 32 + lane);
      bool ready =
          __shfl_sync(0xffffffffu, (int)mbar_wait(acc_full(ab), aphase, abort_flag), 0) != 0;
      if (ready && dual)
        ready = __shfl_sync(0xffffffffu, (int)mbar_wait(acc_full(1), 0u, abort_flag), 0) != 0;
      if (!ready) break;
      tc05_fence_after();
#pragma unroll 1
      for (int c = 0; c < nch; ++c) {
        uint32_t v[32];
        tc05_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + ab * ACC +
                               (uint32_t)(unit * 64 + c * 32), v);
        if (dual) {   // the odd blocks of K
          uint32_t w[32];
          tc05_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + ACC +
                                 (uint32_t)(unit * 64 + c * 32), w);
          tc05_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[j]));
        }
        tc05_wait_ld();
        if (c == nch - 1) {   // this warp has read its share of the accumulator: hand it back
          tc05_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (PAIR)
              asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(
                               lead_empty0 + 8u * ab)
                           : "memory");
            else
              asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(acc_empty(ab)) : "memory");
          }
        }
        const int nb = col0 + c * 32;
        const float bias_l = c == 0 ? bias_pre[0] : bias_pre[1];
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float x = __uint_as_float(v[j]) + __shfl_sync(0xffffffffu, bias_l, j);
          f[j] = nb_apply_act_fast(x, act);
        }
        if constexpr (F32) {
          const uint32_t buf = my_row + c * 4096u;
          if (residual != nullptr) {
            const bool got = __shfl_sync(0xffffffffu,
                                         (int)mbar_wait(res_bar(e, c), t & 1u, abort_flag), 0) != 0;
            if (got) {
#pragma unroll
              for (int q4 = 0; q4 < 8; ++q4) {
                float4 r4;
                asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];\n"
                             : "=f"(r4.x), "=f"(r4.y), "=f"(r4.z), "=f"(r4.w)
                             : "r"(buf + (((uint32_t)q4 ^ swz) << 4)));
                f[4 * q4] += r4.x; f[4 * q4 + 1] += r4.y; f[4 * q4 + 2] += r4.z; f[4 * q4 + 3] += r4.w;
              }
            }
          }
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4)
            asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"r"(buf + (((uint32_t)q4 ^ swz) << 4)),
                         "f"(f[4 * q4]), "f"(f[4 * q4 + 1]), "f"(f[4 * q4 + 2]), "f"(f[4 * q4 + 3])
                         : "memory");
          fence_async_smem();
          __syncwarp();
          if (lane == 0 && nb < N && row0 < M) {
            tma_store_2d(&map_out, stg + c * 4096u, nb, row0);
            bulk_commit();
          }
        } else {
          // 32 columns = four 16-byte pieces of the row's 128 bytes; the second chunk follows
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t p0, p1, p2, p3;
            {
              __nv_bfloat162 h0 = __floats2bfloat162_rn(f[8 * q4], f[8 * q4 + 1]);
              __nv_bfloat162 h1 = __floats2bfloat162_rn(f[8 * q4 + 2], f[8 * q4 + 3]);
              __nv_bfloat162 h2 = __floats2bfloat162_rn(f[8 * q4 + 4], f[8 * q4 + 5]);
              __nv_bfloat162 h3 = __floats2bfloat162_rn(f[8 * q4 + 6], f[8 * q4 + 7]);
              p0 = *reinterpret_cast<uint32_t*>(&h0); p1 = *reinterpret_cast<uint32_t*>(&h1);
              p2 = *reinterpret_cast<uint32_t*>(&h2); p3 = *reinterpret_cast<uint32_t*>(&h3);
            }
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(
                             my_row + ((((uint32_t)(c * 4 + q4)) ^ swz) << 4)),
                         "r"(p0), "r"(p1), "r"(p2), "r"(p3)
                         : "memory");
          }
          if (c == 1) {
            fence_async_smem();
            __syncwarp();
            if (lane == 0 && col0 < N && row0 < M) {
              tma_store_2d(&map_out, stg, col0, row0);
              bulk_commit();
            }
          }
        }
      }
    }
    if (lane == 0) bulk_wait_all();   // stores must have left shared memory before it goes away
  } else {             // ------------------------------------------------------ epilogue, direct stores
    const int quarter = warp & 3;   // the 32 tensor-memory lanes this warp may read
    const int half = (warp - 2) >> 2;   // which share of the tile's columns it takes
    constexpr int CHUNKS = BN / 32 / (EW / 4);   // 32-column chunks per warp
    uint32_t t = 0;
    if (dual) {   // the second issuing thread, before its warp turns to the epilogue
      if (warp == 2 && lane == 0) dual_walk(1);
      __syncwarp();
    }
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t) {
      const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
      const uint32_t ab = t & 1u, aphase = (t >> 1) & 1u;
      // the bias of this warp's columns, fetched while the products still run
      float bias_pre[CHUNKS];
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int nbc = n0 + (half * CHUNKS + c) * 32;
        bias_pre[c] = (bias && nbc + lane < N) ? __ldg(bias + nbc + lane) : 0.0f;
      }
      // lane 0 decides for the warp: the tensor-memory loads below need all 32 lanes
      bool ready =
          __shfl_sync(0xffffffffu, (int)mbar_wait(acc_full(ab), aphase, abort_flag), 0) != 0;
      if (ready && dual)
        ready = __shfl_sync(0xffffffffu, (int)mbar_wait(acc_full(1), 0u, abort_flag), 0) != 0;
      if (!ready) break;
      tc05_fence_after();
#pragma unroll 1
      for (int c = half * CHUNKS; c < (half + 1) * CHUNKS; ++c) {
        uint32_t v[32];
        tc05_ld_32x32b_x32(
            tmem_base + ((uint32_t)(quarter * 32) << 16) + ab * ACC + (uint32_t)(c * 32), v);
        if (dual) {   // the odd blocks of K
          uint32_t w[32];
          tc05_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + ACC + (uint32_t)(c * 32), w);
          tc05_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[j]));
        }
        tc05_wait_ld();
        if (c == (half + 1) * CHUNKS - 1) {   // this warp has read its share: hand it back
          tc05_fence_before();
          __syncwarp();
          if (lane == 0)
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(acc_empty(ab)) : "memory");
        }
        const int nb = n0 + c * 32;
        // bias of the chunk's 32 columns: one value per lane
        float bias_l = bias_pre[0];
#pragma unroll
        for (int q = 1; q < CHUNKS; ++q)
          if (c - half * CHUNKS == q) bias_l = bias_pre[q];
        // The accumulator comes with a lane per row and a register per column; stored that way
        // a warp's instruction would touch 32 rows, four bytes each.  The 32 x 32 block is
        // transposed across the warp (five rounds of exchanges between lanes 16, 8, 4, 2, 1
        // apart), after which lane l holds column l and register i row i: an instruction then
        // writes 32 consecutive columns of one row, whatever the width of the output (the
        // logits' 50,257 columns are no multiple of anything).
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
#pragma unroll
        for (int s2 = 16; s2 >= 1; s2 >>= 1) {
          const bool upper = (lane & s2) != 0;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (j & s2) continue;
            const float send = upper ? f[j] : f[j + s2];
            const float got = __shfl_xor_sync(0xffffffffu, send, s2);
            if (upper) f[j] = got; else f[j + s2] = got;
          }
        }
        const int col = nb + lane;
        const int row0 = m0 + quarter * 32;
        if (col < N) {
          float rs[32];   // `residual` may be `out` itself: all of it before the first store
#pragma unroll
          for (int i = 0; i < 32; ++i)
            rs[i] = (residual && row0 + i < M) ? residual[(size_t)(row0 + i) * N + col] : 0.0f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (row0 + i >= M) break;
            const float y = nb_apply_act_fast(f[i] + bias_l, act) + rs[i];
            if constexpr (sizeof(TOut) == 4) reinterpret_cast<float*>(out)[(size_t)(row0 + i) * N + col] = y;
            else reinterpret_cast<bf16*>(out)[(size_t)(row0 + i) * N + col] = __float2bfloat16_rn(y);
          }
        }
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
  if constexpr (PAIR) {   // neither CTA leaves while the other may still reach into it
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
  }
  if (warp == 1) {
    tc05_fence_after();
    if constexpr (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base),
                   "r"((uint32_t)(2 * ACC))
                   : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base),
                   "r"((uint32_t)(2 * ACC))
                   : "memory");
  }
}

// The word of pinned host memory in which these kernels report a wait that ran out.
int* error_word() {
  int* w = nb_error_words();
  return w ? w + NB_ERRW_GEMM_TCGEN05 : nullptr;
}

// A wait that nothing ends: one thread waits, with the same bounded wait as the kernels above,
// on a barrier that never gets its arrival, and reports the time-out the way they do.  It is
// how a test sees the limit work without any kernel being made to stall.
__global__ void wait_probe_kernel(int* err_word, int* status) {
  __shared__ __align__(8) unsigned long long bar_mem;
  __shared__ int abort_mem;
  const uint32_t bar = smem_u32(&bar_mem);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    abort_mem = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    const bool ok = mbar_wait(bar, 0u, &abort_mem);
    if (!ok) nb_report_timeout(err_word);
    *status = ok ? 1 : 2;
  }
}

// ---------------------------------------------------------------------------------- host
template <int BN, int EPI, typename TOut, int PAIR = 0>
int launch(const void* X, const void* W, const float* bias, const float* residual, void* out, int M,
           int N, int K, int act, cudaStream_t stream) {
  using L = SmemLayout<BN, EPI, (int)sizeof(TOut), PAIR>;
  static_assert(L::STAGES >= 2, "tile shape leaves no room for a pipeline");
  CUtensorMap mx, mw, mo;
  // A product of fewer than 128 rows brings only its rows (in eighths of a tile) into the X
  // part of a stage: the other rows of the MMA's 128 are whatever shared memory holds, and so
  // are their results, which no epilogue stores (rows >= M).  Fewer bytes per K block matter:
  // a single row tile is a stream bound by what one SM can load.
  const int a_rows = M >= BM ? BM : ((M + 15) / 16) * 16;
  int rc = make_map(&mx, X, M, K, a_rows, BK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2);
  if (rc) return rc;
  rc = make_map(&mw, W, N, K, PAIR ? BN / 2 : BN, BK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2);
  if (rc) return rc;
  if (EPI) {
    rc = sizeof(TOut) == 4
             ? make_map(&mo, out, M, N, 32, 32, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4)
             : make_map(&mo, out, M, N, 32, 64, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2);
    if (rc) return rc;
  } else {
    mo = mx;   // unused
  }
  auto kern = gemm_tcgen05_kernel<BN, EPI, TOut, PAIR>;
  const int smem = L::TOTAL;
  static bool configured = false;   // per instantiation
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  constexpr int TILE_M = PAIR ? 2 * BM : BM;
  const int tiles_n = (N + BN - 1) / BN;
  const long long num_tiles = (long long)tiles_n * ((M + TILE_M - 1) / TILE_M);
  NB_REQUIRE(num_tiles < (1ll << 31), NB_ERR_UNSUPPORTED, "gemm_tcgen05: too many tiles");
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    NB_CUDA(cudaGetDevice(&dev));
    NB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  }
  if constexpr (PAIR) {
    // clusters of two CTAs, one cluster per pair of SMs
    const int pairs = (int)(num_tiles < sms / 2 ? num_tiles : sms / 2);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(cta_threads(BN, EPI));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    NB_CUDA(cudaLaunchKernelEx(&cfg, kern, mx, mw, mo, bias, residual, (TOut*)out, M, N, K, act, tiles_n,
                               (int)num_tiles, a_rows * BK * 2, error_word(), 0));
    return 0;
  }
  const int grid = (int)(num_tiles < sms ? num_tiles : sms);   // one CTA per SM walks the tiles
  // Several producer lanes only for a single row tile (a decode step, a short prompt): its
  // boxes are small and the producer's issue rate bounds the kernel.  With large tiles the
  // MMAs bound it, and lanes that fill the ring out of order only delay the stage the MMAs
  // wait for (a 2,048-token prefill: 1.16 -> 1.28 ms with four lanes); there one lane brings X
  // and one W, both in order (the kernel's `split_xw`).
  const int tune = (g_dual ? 1 : 0) | ((g_lanes ? (M <= BM ? 2 : 1) : 0) << 1);
  NB_CUDA(nb_launch(kern, dim3(grid), dim3(cta_threads(BN, EPI)), (size_t)smem, stream, mx, mw, mo, bias,
                    residual, (TOut*)out, M, N, K, act, tiles_n, (int)num_tiles, a_rows * BK * 2,
                    error_word(), tune));
  return 0;
}

// Tile width.  A single row tile (at most 128 rows) is a weight stream: many narrow tiles
// with a deep ring.  Otherwise every tile re-reads its 128 rows of X and its BN rows of W from
// L2, so wide tiles win for large products; for products of a few hundred tiles what counts
// is how many waves the 148 SMs need and how long a wave is, so the width is the one with
// the least waves x (width + a tile's fixed cost, about 48 columns' worth of time).  The
// fp32 TMA epilogue has room for 128 columns at most and alone takes 96; the direct-store
// epilogue takes 64, 128 and 256.
int pick_tile_width(int M, int N, bool f32_out, bool tma_epi) {
  const long long tiles_m = (M + BM - 1) / BM;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  // A single row tile: narrow tiles, so that many CTAs share the stream of weights -- unless
  // there are more of them than SMs (the output head): an MMA costs its issuing thread the
  // same up to 128 columns, so a CTA that walks over several tiles does so twice as fast with
  // tiles of 128.
  if (tiles_m == 1) return (N + 63) / 64 > sms ? 128 : 64;
  const int cand_f32_tma[] = {128, 96, 64}, cand_bf16_tma[] = {256, 192, 128, 64}, cand_direct[] = {256, 128, 64};
  const int* cand = !tma_epi ? cand_direct : (f32_out ? cand_f32_tma : cand_bf16_tma);
  const int n_cand = !tma_epi ? 3 : (f32_out ? 3 : 4);
  int best = cand[n_cand - 1];
  long long best_cost = -1;
  for (int i = 0; i < n_cand; ++i) {
    const int bn = cand[i];
    if (bn > 64 && N < bn) continue;                       // wider than the output: wasted columns
    const long long tiles = tiles_m * ((N + bn - 1) / bn);
    const long long cost = ((tiles + sms - 1) / sms) * (bn + 48);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }   // ties: the wider
  }
  return best;
}

// What a large product is bound by is the 64 bytes per clock an SM can take in: a 128 x 256
// tile brings 48 KB per K block for 512 clocks of MMAs.  In a pair each CTA brings half of the
// weight tile (32 KB), which measures 1.36 against 1.20 PFLOP/s at 8192 x 6400 x 1600.  A
// product of a wave or two of tiles is no faster in pairs, or slower (12.3 -> 13.4 us at
// 2048 x 2304 x 768): the cluster's start-up and its barriers cost more than the lighter
// loads save; pairs are taken from three waves of single-CTA tiles on.
int g_use_pairs = 1;   // 0 off, 1 where the cost model prefers them, 2 wherever a paired kernel exists

// Width of 256-row tiles for pairs of CTAs, or 0 if single CTAs with `single_bn` are better.
// Cost of a shape: waves over the SMs (or pairs of SMs) x what a CTA brings in per K block
// (its rows of X, its rows of W) plus a tile's fixed cost, all in rows of 128 bytes.
int pick_pair_width(int M, int N, bool f32_out, int single_bn) {
  if (M <= BM) return 0;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  const long long fixed = 64;
  const long long tiles1 = (long long)((M + BM - 1) / BM) * ((N + single_bn - 1) / single_bn);
  // measured: pairs pay from three waves of single-CTA tiles on, for narrow outputs (fewer
  // than 1024 columns) from six
  if (g_use_pairs < 2 && (tiles1 < 3ll * sms || (N < 1024 && tiles1 < 6ll * sms))) return 0;
  long long best_cost = g_use_pairs >= 2 ? (1ll << 60)
                                         : ((tiles1 + sms - 1) / sms) * (BM + single_bn + fixed);
  int best = 0;
  const int cand_f32[] = {128, 96}, cand_bf16[] = {256, 192, 128};
  const int* cand = f32_out ? cand_f32 : cand_bf16;
  const int n_cand = f32_out ? 2 : 3;
  const int pairs = sms / 2;
  for (int i = 0; i < n_cand; ++i) {
    const int bn = cand[i];
    if (N < bn && i + 1 < n_cand) continue;               // wider than the output: try a narrower one
    const long long tiles2 = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + bn - 1) / bn);
    const long long cost = ((tiles2 + pairs - 1) / pairs) * (BM + bn / 2 + fixed);
    if (cost < best_cost) { best_cost = cost; best = bn; }
  }
  return best;
}

}  // namespace

// 1 if the tensor-core kernel takes this product.
NB_EXPORT int nb_gemm_tcgen05_supported(int x_dtype, int w_dtype, int M, int N, int K) {
  return x_dtype == NB_BF16 && w_dtype == NB_BF16 && K % 8 == 0 && M >= 1 && N >= 1 && K >= 8 &&
         (M + BM - 1) / BM <= 65535;
}

// Comparison runs: two MMA-issuing threads on or off, several producer lanes on or off.
NB_EXPORT int nb_gemm_tcgen05_tune(int dual, int lanes) {
  g_dual = dual != 0;
  g_lanes = lanes != 0;
  return 0;
}

// Pairs of CTAs on 256-row tiles: 0 never, 1 where the cost model prefers them, 2 wherever a
// paired kernel exists.
NB_EXPORT int nb_gemm_tcgen05_use_pairs(int mode) {
  g_use_pairs = mode < 0 ? 0 : (mode > 2 ? 2 : mode);
  return 0;
}

// Waits for the device, then reads (and lowers) the word that a timed-out wait of these kernels
// raises.
NB_EXPORT int nb_gemm_tcgen05_error() {
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  volatile int* w = error_word();
  if (w == nullptr) return 0;
  const int v = *w;
  if (v) *w = 0;
  return v;
}

// Clock cycles a wait of these kernels may take before it gives up (default 4e9, about two
// seconds).  Takes effect for kernels launched after the call.
NB_EXPORT int nb_gemm_tcgen05_set_wait_budget(long long cycles) {
  NB_REQUIRE(cycles >= 0, NB_ERR_BAD_ARG, "wait budget must not be negative");
  return set_wait_budget(cycles);
}

// Runs the bounded wait on a barrier that nothing completes: `status` (device int) receives 2
// when the wait gave up after the budget (and the probe's error word is raised), 1 if it came
// back complete.
NB_EXPORT int nb_wait_probe(int* status, cudaStream_t stream) {
  int* w = nb_error_words();
  wait_probe_kernel<<<1, 32, 0, stream>>>(w ? w + NB_ERRW_PROBE : nullptr, status);
  NB_CHECK_LAUNCH("wait_probe");
  return 0;
}

NB_EXPORT int nb_gemm_tcgen05(const void* X, const void* W, const float* bias, const float* residual,
                              void* out, int out_dtype, int M, int N, int K, int act,
                              cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  NB_REQUIRE(nb_gemm_tcgen05_supported(NB_BF16, NB_BF16, M, N, K), NB_ERR_UNSUPPORTED,
             "gemm_tcgen05: needs bf16 operands and a width that is a multiple of 8 (M=%d N=%d K=%d)",
             M, N, K);
  NB_REQUIRE((uintptr_t)X % 16 == 0 && (uintptr_t)W % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                 (uintptr_t)residual % 16 == 0,
             NB_ERR_UNSUPPORTED, "gemm_tcgen05: operands must be 16-byte aligned");
  // Epilogue through shared memory and TMA stores (full-line writes, residual fetched by TMA)
  // when the output rows are 16-byte multiples and the residual, if any, is the output
  // itself; otherwise every thread stores its own row segment.
  const int esize = out_dtype == NB_F32 ? 4 : 2;
  const bool tma_epi = ((long long)N * esize) % 16 == 0 && (residual == nullptr || residual == out);
  const int bn = pick_tile_width(M, N, out_dtype == NB_F32, tma_epi);
  int rc;
  // Pairs of CTAs on 256-row tiles bring less into each SM per flop (half of the weight tile
  // each); they are taken when that outweighs the coarser tiles (see pick_pair_width).
  const int pair_bn = (tma_epi && g_use_pairs) ? pick_pair_width(M, N, out_dtype == NB_F32, bn) : 0;
  if (pair_bn) {
    rc = NB_ERR_BAD_ARG;
    if (out_dtype == NB_F32) {
      if (pair_bn == 128) rc = launch<128, 1, float, 1>(X, W, bias, residual, out, M, N, K, act, stream);
      else if (pair_bn == 96) rc = launch<96, 1, float, 1>(X, W, bias, residual, out, M, N, K, act, stream);
    } else if (out_dtype == NB_BF16) {
      if (pair_bn == 256) rc = launch<256, 1, bf16, 1>(X, W, bias, residual, out, M, N, K, act, stream);
      else if (pair_bn == 192) rc = launch<192, 1, bf16, 1>(X, W, bias, residual, out, M, N, K, act, stream);
      else if (pair_bn == 128) rc = launch<128, 1, bf16, 1>(X, W, bias, residual, out, M, N, K, act, stream);
    }
    NB_REQUIRE(rc != NB_ERR_BAD_ARG, NB_ERR_BAD_ARG, "gemm_tcgen05: no paired kernel of width %d", pair_bn);
    if (rc) return rc;
    NB_CHECK_LAUNCH("gemm_tcgen05");
    return 0;
  }
#define NB_TC(BN_, EPI_, T_) rc = launch<BN_, EPI_, T_>(X, W, bias, residual, out, M, N, K, act, stream)
  if (out_dtype == NB_F32) {
    if (tma_epi) {
      if (bn == 128) NB_TC(128, 1, float); else if (bn == 96) NB_TC(96, 1, float); else NB_TC(64, 1, float);
    } else {
      if (bn == 256) NB_TC(256, 0, float); else if (bn == 128) NB_TC(128, 0, float); else NB_TC(64, 0, float);
    }
  } else if (out_dtype == NB_BF16) {
    if (tma_epi) {
      if (bn == 256) NB_TC(256, 1, bf16); else if (bn == 192) NB_TC(192, 1, bf16);
      else if (bn == 128) NB_TC(128, 1, bf16); else NB_TC(64, 1, bf16);
    } else {
      if (bn == 256) NB_TC(256, 0, bf16); else if (bn == 128) NB_TC(128, 0, bf16); else NB_TC(64, 0, bf16);
    }
  } else {
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "gemm_tcgen05: unknown output dtype %d", out_dtype);
  }
#undef NB_TC
  if (rc) return rc;
  NB_CHECK_LAUNCH("gemm_tcgen05");
  return 0;
}
