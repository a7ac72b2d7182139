// Matrix product for 17 to 128 rows (a decode step of a larger batch, a short prompt) on the
// 5th-generation tensor cores: out[M,N] = act(X[M,K] * W[N,K]^T + bias) (+ residual), bf16
// operands, fp32 accumulation in tensor memory.
//
// What bounds such a product is not the tensor cores but the thread that feeds them: one
// `tcgen05.mma` costs its issuing thread about 80 clocks whatever its width up to 128 columns
// (measured on a B200: 81 clocks an instruction at N = 32, 64 and 128, 142 at N = 256).  So the
// kernel makes every instruction cover as many weights as it can and gives every CTA few of
// them:
//   * the operands are swapped: the weights are the 128-row operand (A), the step's rows the
//     narrow one (B, N = rows rounded up to 16), so an instruction covers 128 weight rows
//     whatever the number of rows of X -- the accumulator is the product's transpose, 128
//     weight rows (tensor-memory lanes) x rows of X (columns);
//   * K is cut among the CTAs of a thread-block cluster (1 to 8), chosen so that the launch
//     fills the GPU once: each CTA walks over its run of 64-column blocks of K into its own
//     accumulator;
//   * the sums meet by a reduce-scatter through distributed shared memory: the rows of X are
//     dealt out to the CTAs of the cluster (in fours), every CTA sends each other CTA that
//     CTA's rows of its accumulator with `st.async` (16 bytes a store, counted on a barrier in
//     the receiver's shared memory, so no cluster barrier stands between sending and adding
//     up), and each adds up what it got in rank order (the result does not depend on timing),
//     applies bias, activation and residual and stores its rows: 32 lanes write 32
//     consecutive columns of a row.
// Warp 0: one thread issues the TMA loads (128 x 64 boxes of W, rows x 64 boxes of X, 128-byte
// swizzled) into a ring of stages; the weights of the first stages are asked for before the
// wait on the kernel in front (they are constants).  Warp 1 owns the tensor memory and issues
// the MMAs.  Warps 2 to 5 are the epilogue, one per quarter of the lanes.
//
// Every wait on an mbarrier is bounded by a clock budget; a wait that runs out raises the
// kernel's error word, all roles leave their loops, every thread still passes the cluster's
// barriers (a hardware barrier has no limit of its own, so nobody may skip it), the CTA frees
// its tensor memory and returns.
//
// Requirements: K % 8 == 0 (16-byte row pitch for TMA), 16-byte aligned bases, N at most
// 128 x the number of SMs.  Reference analogue: Mat::gemm_into (src/model.rs:94-133).
#include "tc05_common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

constexpr int BW = 128;              // weight rows per tile = rows of the MMA
constexpr int BK = 64;               // 64 bf16 = 128 bytes = one swizzle atom row
constexpr int UMMA_K = 16;
constexpr int MAX_ROWS = 128;
constexpr int MAX_STAGES = 8;
constexpr int MAX_SPLIT = 8;         // portable cluster size
constexpr int W_BYTES = BW * BK * 2;                 // 16 KB
constexpr int THREADS = 64 + 4 * 32;
constexpr int SMEM_BUDGET = 200 * 1024;

struct RowsShape {
  int nb;            // rows of X rounded up to 16: the MMA's N
  int split;         // CTAs of a cluster = runs of K
  int kb_per;        // K blocks per CTA
  int stages;        // stages of the ring
  int stage_bytes;   // W box + X box
  int x_bytes;       // X box
  int chunk;         // rows of X a CTA finishes (a multiple of 4)
  int cpad;          // floats between two weight rows in the receive buffer (cpad / 4 is odd)
  int tmem_cols;     // power of two >= nb, >= 32
  int smem;          // dynamic shared memory
};

// Four rows of the residual at column n (zero where there is none).
__device__ __forceinline__ void load_residual4(float (&r)[4], const float* residual, int m0, int m_end,
                                               int n, int N) {
#pragma unroll
  for (int j = 0; j < 4; ++j)
    r[j] = (residual && m0 + j < m_end) ? residual[(size_t)(m0 + j) * N + n] : 0.0f;
}

__device__ __forceinline__ void st_async_v4(uint32_t remote, uint32_t remote_bar, const uint32_t* v) {
  asm volatile(
      "st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1,%2,%3,%4}, [%5];\n" ::"r"(remote),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(remote_bar)
      : "memory");
}

// One row of the result: bias, activation, residual, store.
template <typename TOut>
__device__ __forceinline__ void finish_rows4(const float (&a)[4], const float (&r)[4], int m0, int m_end,
                                             int n, int N, float b, int act, TOut* out) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (m0 + j >= m_end) break;
    const float y = nb_apply_act_fast(a[j] + b, act) + r[j];
    if constexpr (sizeof(TOut) == 4) reinterpret_cast<float*>(out)[(size_t)(m0 + j) * N + n] = y;
    else reinterpret_cast<bf16*>(out)[(size_t)(m0 + j) * N + n] = __float2bfloat16_rn(y);
  }
}

template <typename TOut>
__global__ void __launch_bounds__(THREADS)
gemm_tc_rows_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const float* __restrict__ bias, const float* residual, TOut* out, int M, int N,
                    int K, int act, RowsShape sh, int* err_word) {
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;          // swizzle atoms want 1024-byte alignment
  unsigned char* gen = smem_dyn + (base - raw);
  // [ring of stages] [what the other CTAs send: [rank][128 weight rows][cpad]] [barriers]
  // [tmem slot, abort]
  const uint32_t ring_bytes = (uint32_t)(sh.stages * sh.stage_bytes);
  const uint32_t recv = base + ring_bytes;
  const uint32_t recv_bytes = sh.split > 1 ? (uint32_t)(sh.split * BW * sh.cpad * 4) : 0u;
  const uint32_t bars = recv + recv_bytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (MAX_STAGES + s); };
  const uint32_t acc_full = bars + 8u * (2 * MAX_STAGES);
  const uint32_t recv_bar = bars + 8u * (2 * MAX_STAGES + 1);
  uint32_t* tmem_slot =
      reinterpret_cast<uint32_t*>(gen + ring_bytes + recv_bytes + (2 * MAX_STAGES + 2) * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
  const int n0 = (int)(blockIdx.x / sh.split) * BW;
  const int num_kb = (K + BK - 1) / BK;
  const int kb_lo = (int)rank * sh.kb_per, kb_hi = min(num_kb, kb_lo + sh.kb_per);
  const int n_kb = max(0, kb_hi - kb_lo);

  if (tid == 0) {
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
    for (int s = 0; s < sh.stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(recv_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"((uint32_t)sh.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc05_fence_before();
  __syncthreads();
  tc05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // The weights of the first stages are constants: they are asked for while the kernel in
  // front is still running.  Nothing that concerns the cluster happens before the wait.
  int pre_kb = 0;
  if (tid == 0) {
    pre_kb = min(n_kb, sh.stages);
    for (int i = 0; i < pre_kb; ++i) {
      mbar_expect_tx(full_bar(i), (uint32_t)sh.stage_bytes);
      tma_load_2d(base + i * sh.stage_bytes, &map_w, (kb_lo + i) * BK, n0, full_bar(i));
    }
  }
  nb_grid_dependency_wait();
  // Rows of X this CTA finishes, and the bytes the other CTAs will send for them.
  const int m_lo = (int)rank * sh.chunk;
  const int my_rows = max(0, min(sh.nb, m_lo + sh.chunk) - m_lo);
  if (tid == 0 && sh.split > 1)
    mbar_expect_tx(recv_bar, (uint32_t)((sh.split - 1) * BW * my_rows * 4));
  // Every CTA of the cluster says that it runs and that its barrier is armed; the matching
  // wait stands in front of the first store into another CTA's shared memory, by when the
  // others have long arrived.  (The arrive stands behind the wait on the predecessor: see
  // the decode attention.)
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");

  if (warp == 0) {
    // A TMA tile load costs its issuing thread about 190 clocks whatever the size of its box:
    // up to four lanes, each with every n-th block of K, keep the TMA unit busy.  Their number
    // divides the number of stages, so a lane owns its stages and fills one again only after
    // its own earlier wait for it: it can never be two rounds of the ring ahead of the MMAs
    // (where the parity of an older phase of the stage's barrier would pass for the awaited one).
    pre_kb = __shfl_sync(0xffffffffu, pre_kb, 0);
    const int producers = sh.stages % 4 == 0 ? 4 : (sh.stages % 3 == 0 ? 3 : (sh.stages % 2 == 0 ? 2 : 1));
    if (lane < producers) {   // --------------------------------------------- TMA producers
      for (int i = lane; i < n_kb; i += producers) {
        const int s = i % sh.stages;
        const uint32_t dst = base + s * sh.stage_bytes;
        if (i < pre_kb) {   // armed, and its weights on their way: the rows follow
          tma_load_2d(dst + W_BYTES, &map_x, (kb_lo + i) * BK, 0, full_bar(s));
          continue;
        }
        if (!mbar_wait(empty_bar(s), ((i / sh.stages) & 1u) ^ 1u, abort_flag)) break;
        mbar_expect_tx(full_bar(s), (uint32_t)sh.stage_bytes);
        tma_load_2d(dst + W_BYTES, &map_x, (kb_lo + i) * BK, 0, full_bar(s));
        tma_load_2d(dst, &map_w, (kb_lo + i) * BK, n0, full_bar(s));
      }
      nb_launch_dependents();   // every load is on its way
    }
  } else if (warp == 1) {
    if (lane == 0) {   // ------------------------------------------------------ MMA issuer
      const uint32_t idesc = instr_desc_bf16(BW, sh.nb);
      bool ok = true;
      for (int i = 0; i < n_kb && ok; ++i) {
        const int s = i % sh.stages;
        ok = mbar_wait(full_bar(s), (i / sh.stages) & 1u, abort_flag);
        if (!ok) break;
        tc05_fence_after();
        const uint32_t w_addr = base + s * sh.stage_bytes;
        const uint64_t da = smem_desc_sw128(w_addr);
        const uint64_t db = smem_desc_sw128(w_addr + W_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)   // 16 elements of K = 32 bytes = 2 address units
          tc05_mma_bf16(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                        (i > 0 || k > 0) ? 1u : 0u);
        if (i + sh.stages < n_kb) tc05_commit(empty_bar(s));   // only a stage that is used again
      }
      if (ok) {
        if (n_kb > 0) tc05_commit(acc_full);
        else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(acc_full) : "memory");
      }
    }
  }

  // ---- epilogue warps: this CTA's sums are complete
  const int quarter = warp & 3;                 // the 32 tensor-memory lanes this warp may read
  const int n_local = quarter * 32 + lane;      // weight row of the tile = column of the output
  const int n = n0 + n_local;
  const int m_end = min(M, sh.nb);
  // the bias of this thread's column (a constant), fetched while the products run
  const float b = (warp >= 2 && bias && n < N) ? __ldg(bias + n) : 0.0f;
  bool ready = true;
  if (warp >= 2)
    ready = __shfl_sync(0xffffffffu, (int)mbar_wait(acc_full, 0u, abort_flag), 0) != 0;
  // the lanes of the producer's and the issuer's warps come together first: the barrier wants
  // whole warps
  __syncwarp();
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");

  if (warp >= 2 && ready) {
    tc05_fence_after();
    // columns of the accumulator = rows of X, in fours; four that belong to CTA d go to
    // [this rank][n_local][their place in d's rows] of d's buffer, the own ones stay here
    const uint32_t slot = recv + (uint32_t)(((int)rank * BW + n_local) * sh.cpad) * 4u;
    for (int c0 = 0; c0 < sh.nb; c0 += 32) {
      uint32_t v[32];
      if (n_kb > 0) {
        tc05_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
        tc05_wait_ld();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0u;
      }
      if (sh.split == 1) {   // nothing to exchange: finish the rows right away
        if (n < N) {
          // all of the chunk's residual before its first store: it may be `out` itself, and a
          // load behind a store would wait for it
          float res[8][4];
#pragma unroll
          for (int g4 = 0; g4 < 8; ++g4) load_residual4(res[g4], residual, c0 + 4 * g4, m_end, n, N);
#pragma unroll
          for (int g4 = 0; g4 < 8; ++g4) {
            if (c0 + 4 * g4 >= m_end) break;
            const float a[4] = {__uint_as_float(v[4 * g4]), __uint_as_float(v[4 * g4 + 1]),
                                __uint_as_float(v[4 * g4 + 2]), __uint_as_float(v[4 * g4 + 3])};
            finish_rows4<TOut>(a, res[g4], c0 + 4 * g4, m_end, n, N, b, act, out);
          }
        }
        continue;
      }
#pragma unroll
      for (int g4 = 0; g4 < 8; ++g4) {
        const int m = c0 + 4 * g4;
        if (m >= sh.nb) break;
        const int dest = m / sh.chunk;
        const uint32_t at = slot + (uint32_t)(m - dest * sh.chunk) * 4u;
        if (dest == (int)rank) {
          asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(at), "r"(v[4 * g4]), "r"(v[4 * g4 + 1]),
                       "r"(v[4 * g4 + 2]), "r"(v[4 * g4 + 3])
                       : "memory");
        } else {
          st_async_v4(cluster_addr(at, (uint32_t)dest), cluster_addr(recv_bar, (uint32_t)dest), &v[4 * g4]);
        }
      }
    }
    tc05_fence_before();
  }
  // Second phase of the cluster's barrier: this thread has sent what it had to send (the wait
  // is the last thing the kernel does: no CTA leaves while another may still send to it).
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  if (warp >= 2 && ready) {
    if (sh.split > 1) {
      // the residual of this CTA's first rows is fetched while the others' sums are on their way
      constexpr int PRE = 4;
      float res[PRE][4];
#pragma unroll
      for (int g4 = 0; g4 < PRE; ++g4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) res[g4][j] = 0.0f;
        if (n < N && 4 * g4 < my_rows) load_residual4(res[g4], residual, m_lo + 4 * g4, m_end, n, N);
      }
      // what the others sent for this CTA's rows has arrived when the barrier has its bytes
      const bool got = __shfl_sync(0xffffffffu, (int)mbar_wait(recv_bar, 0u, abort_flag), 0) != 0;
      if (got && n < N) {
        for (int off0 = 0; off0 < my_rows; off0 += 4 * PRE) {
          if (off0 > 0) {   // further rows: their residual now, all of it before the next stores
#pragma unroll
            for (int g4 = 0; g4 < PRE; ++g4)
              if (off0 + 4 * g4 < my_rows) load_residual4(res[g4], residual, m_lo + off0 + 4 * g4, m_end, n, N);
          }
#pragma unroll
          for (int g4 = 0; g4 < PRE; ++g4) {
            const int off = off0 + 4 * g4;
            if (off >= my_rows || m_lo + off >= m_end) break;
            float a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int s = 0; s < sh.split; ++s) {   // in rank order
              float4 x;
              asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];\n"
                           : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w)
                           : "r"(recv + (uint32_t)((s * BW + n_local) * sh.cpad + off) * 4u));
              a[0] += x.x; a[1] += x.y; a[2] += x.z; a[3] += x.w;
            }
            finish_rows4<TOut>(a, res[g4], m_lo + off, m_end, n, N, b, act, out);
          }
        }
      }
    }
  }

  __syncwarp();
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
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
                 "r"((uint32_t)sh.tmem_cols)
                 : "memory");
  }
}

int* error_word() {
  int* w = nb_error_words();
  return w ? w + NB_ERRW_GEMM_TC_ROWS : nullptr;
}

int device_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  return sms;
}

int g_force_split = 0;   // tuning and tests: 0 = choose

// How the product is laid out, or false if this kernel does not take it.  The cluster size is
// the one with the shortest walk per CTA (the larger of what its MMAs cost the issuing thread
// and what its loads cost the SM's 64 bytes a clock) plus what a cluster costs, among those
// that put the whole launch on the GPU at once.
bool plan_rows(int M, int N, int K, RowsShape* out) {
  if (M < 1 || M > MAX_ROWS || N < 1 || K < 8 || K % 8 != 0) return false;
  const int sms = device_sms();
  const int tiles_n = (N + BW - 1) / BW;
  if (tiles_n > sms) return false;
  RowsShape s;
  s.nb = (M + 15) / 16 * 16;
  s.x_bytes = s.nb * BK * 2;
  s.stage_bytes = W_BYTES + s.x_bytes;
  s.tmem_cols = s.nb <= 32 ? 32 : (s.nb <= 64 ? 64 : 128);
  const int num_kb = (K + BK - 1) / BK;
  long long best_cost = -1;
  int best = 1;
  for (int split = 1; split <= MAX_SPLIT; ++split) {
    if (g_force_split && split != g_force_split) continue;
    if (tiles_n * split > sms && split > 1) break;
    const int kb_per = (num_kb + split - 1) / split;
    if (split > 1 && (split - 1) * kb_per >= num_kb) continue;   // a CTA without a K block
    const long long mma = (long long)kb_per * (BK / UMMA_K) * 85;
    const long long load = (long long)kb_per * s.stage_bytes / 64;
    const long long cost = (mma > load ? mma : load) + (split > 1 ? 600 : 0) + 40LL * split;
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = split; }
  }
  if (best_cost < 0) return false;
  s.split = best;
  s.kb_per = (num_kb + best - 1) / best;
  s.chunk = ((s.nb + best - 1) / best + 3) / 4 * 4;
  s.cpad = (s.chunk / 4) % 2 == 1 ? s.chunk : s.chunk + 4;   // an odd number of 16-byte units: no bank conflicts
  const int recv = best > 1 ? best * BW * s.cpad * 4 : 0;
  int stages = s.kb_per < MAX_STAGES ? s.kb_per : MAX_STAGES;
  while (stages > 1 && stages * s.stage_bytes + recv > SMEM_BUDGET) --stages;
  s.stages = stages;
  s.smem = stages * s.stage_bytes + recv + (2 * MAX_STAGES + 2) * 8 + 16 + 1024;
  if (s.smem > 227 * 1024) return false;
  *out = s;
  return true;
}

template <typename TOut>
int launch_rows(const void* X, const void* W, const float* bias, const float* residual, void* out,
                int M, int N, int K, int act, const RowsShape& sh, cudaStream_t stream) {
  CUtensorMap mx, mw;
  int rc = make_map(&mx, X, M, K, sh.nb, BK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2);
  if (rc) return rc;
  rc = make_map(&mw, W, N, K, BW, BK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2);
  if (rc) return rc;
  auto kern = gemm_tc_rows_kernel<TOut>;
  static bool configured = false;   // per instantiation
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured = true;
  }
  const int tiles_n = (N + BW - 1) / BW;
  NB_CUDA(nb_launch_clusters(kern, dim3(tiles_n * sh.split), dim3(THREADS), (size_t)sh.smem, stream,
                             sh.split, mx, mw, bias, residual, (TOut*)out, M, N, K, act, sh,
                             error_word()));
  return 0;
}

}  // namespace

// 1 if this kernel takes the product.
NB_EXPORT int nb_gemm_tc_rows_supported(int M, int N, int K) {
  RowsShape sh;
  return plan_rows(M, N, K, &sh) ? 1 : 0;
}

// 1 where this kernel is the faster one of the two tensor-core products (measured on a B200 at
// 32, 64 and 128 rows on GPT-2 124M's and XL's shapes): a long K (24 blocks and more) over
// few columns, where the tiled kernel has few CTAs and each a long walk.  Elsewhere the
// exchange between the CTAs of a cluster (about 8 bytes a clock and SM) costs more than the
// shorter walk saves.
NB_EXPORT int nb_gemm_tc_rows_preferred(int M, int N, int K) {
  RowsShape sh;
  if (!plan_rows(M, N, K, &sh)) return 0;
  const int num_kb = (K + BK - 1) / BK;
  return num_kb >= 24 && N <= 74 * 64 && (M <= 96 || num_kb >= 48);
}

// The layout chosen for a shape (tests and reports): nb, split, kb_per, stages, chunk, smem.
NB_EXPORT int nb_gemm_tc_rows_plan(int M, int N, int K, int* out6) {
  RowsShape sh;
  if (!plan_rows(M, N, K, &sh)) return 0;
  out6[0] = sh.nb; out6[1] = sh.split; out6[2] = sh.kb_per; out6[3] = sh.stages; out6[4] = sh.chunk;
  out6[5] = sh.smem;
  return 1;
}

// Tuning and tests: the cluster size to use (0 = choose).  Returns the earlier setting.
NB_EXPORT int nb_gemm_tc_rows_force_split(int split) {
  const int was = g_force_split;
  g_force_split = split < 0 ? 0 : (split > MAX_SPLIT ? MAX_SPLIT : split);
  return was;
}

NB_EXPORT int nb_gemm_tc_rows_set_wait_budget(long long cycles) { return set_wait_budget(cycles); }

NB_EXPORT int nb_gemm_tc_rows(const void* X, const void* W, const float* bias, const float* residual,
                              void* out, int out_dtype, int M, int N, int K, int act,
                              cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  RowsShape sh;
  NB_REQUIRE(plan_rows(M, N, K, &sh), NB_ERR_UNSUPPORTED,
             "gemm_tc_rows: takes 1 to %d rows, K a multiple of 8 and at most %d columns (M=%d N=%d K=%d)",
             MAX_ROWS, BW * device_sms(), M, N, K);
  NB_REQUIRE((uintptr_t)X % 16 == 0 && (uintptr_t)W % 16 == 0, NB_ERR_UNSUPPORTED,
             "gemm_tc_rows: operands must be 16-byte aligned");
  int rc;
  if (out_dtype == NB_F32)
    rc = launch_rows<float>(X, W, bias, residual, out, M, N, K, act, sh, stream);
  else if (out_dtype == NB_BF16)
    rc = launch_rows<bf16>(X, W, bias, residual, out, M, N, K, act, sh, stream);
  else
    NB_REQUIRE(false, NB_ERR_BAD_ARG, "gemm_tc_rows: unknown output dtype %d", out_dtype);
  if (rc) return rc;
  NB_CHECK_LAUNCH("gemm_tc_rows");
  return 0;
}
