// Matrix products with few rows (a decode step: one row per sequence, at most 64):
// out[M,N] = act(norm?(X)[M,K] * W[N,K]^T + bias) (+ residual).
//
// With so few rows the product is bound by streaming W once from HBM, and for a small model
// by latency.  Each CTA owns 8 output columns and all rows; its warps split K, every lane
// fetches its part of the 8 weight rows with 16-byte loads straight into registers, all in
// flight at once, and the tensor cores (mma.sync m16n8k16, bf16 in, fp32 accumulate) do the
// arithmetic; partial sums of the warps are added through shared memory.  The LayerNorm that
// precedes the product in a pre-norm block can be applied while the weights are in flight
// (statistics in fp32, src/ops.rs:32-40), which saves a kernel and a round trip of the
// normalised rows.  A second kernel does the same job with fp32 weights on the CUDA cores
// (true 32-bit path).
//
// Reference analogue: Mat::gemv_into (src/model.rs:65-86), one dot product per output.
#include "common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Eight consecutive elements of a row as floats (16-byte loads; the row start and k are
// multiples of 8 elements).
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __bfloat162float(h[i].x);
    v[2 * i + 1] = __bfloat162float(h[i].y);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return u;
}

// CH, a template parameter of the kernel: the 32-wide K chunks whose weights a warp holds in
// registers at a time (12 for long rows, 4 when that covers a whole row: fewer registers, so
// that two CTAs fit on an SM).
constexpr int VMAX = 8;  // most 8-element vectors of a row a thread may hold while it is normalised

// Sum of `v` over the `tpr` consecutive threads that share a row (tpr is a multiple of 32 and
// divides the block).  `part` holds one float per warp.  Every thread of the block calls it.
__device__ __forceinline__ float row_group_sum(float v, float* part, int tid, int tpr) {
  v = nb_warp_sum(v);
  if (tpr == 32) return v;
  __syncthreads();
  if ((tid & 31) == 0) part[tid >> 5] = v;
  __syncthreads();
  const int first = (tid / tpr) * (tpr >> 5);
  float s = 0.0f;
  for (int w = 0; w < (tpr >> 5); ++w) s += part[first + w];
  return s;
}

// Rows of X, LayerNorm applied, into shared memory as bf16 -- all threads of the block share
// the work of every row: a row belongs to `tpr` consecutive threads, each thread holds its
// vectors of the row in registers (one trip to memory for the row, the norm's weight and its
// bias together), mean and variance are reduced over the row's threads (two passes over the
// registers, src/ops.rs:32-40).  Needs K <= 8 * tpr * VPT; only the M real rows are written.
template <int NT, int VPT>
__device__ __forceinline__ void stage_rows_norm(const float* X, bf16* xs, int stride,
                                                int M, int K, int width,
                                                const float* __restrict__ gamma,
                                                const float* __restrict__ beta, float eps,
                                                float* part, int tid, int tpr) {
  const int rows_per_pass = NT / tpr;
  const int tr = tid % tpr;
  for (int r0 = 0; r0 < M; r0 += rows_per_pass) {
    const int r = r0 + tid / tpr;
    const bool live = r < M;
    const float* src = X + (size_t)(live ? r : 0) * K;
    float v[VPT][8];
    uint4 gm_raw[VPT][2], bt_raw[VPT][2];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int k = (tr + i * tpr) * 8;
      if (live && k < K) {
        load8(src + k, v[i]);
        gm_raw[i][0] = __ldg(reinterpret_cast<const uint4*>(gamma + k));
        gm_raw[i][1] = __ldg(reinterpret_cast<const uint4*>(gamma + k + 4));
        if (beta) {
          bt_raw[i][0] = __ldg(reinterpret_cast<const uint4*>(beta + k));
          bt_raw[i][1] = __ldg(reinterpret_cast<const uint4*>(beta + k + 4));
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = 0.0f;
      }
    }
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int e = 0; e < 8; ++e) s += v[i][e];
    const float mean = row_group_sum(s, part, tid, tpr) / (float)K;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      if (live && (tr + i * tpr) * 8 < K) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float c = v[i][e] - mean;
          q = fmaf(c, c, q);
        }
      }
    }
    const float inv = 1.0f / sqrtf(row_group_sum(q, part, tid, tpr) / (float)K + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int k = (tr + i * tpr) * 8;
      if (!live || k >= width) continue;
      if (k < K) {
        const float* gm = reinterpret_cast<const float*>(&gm_raw[i][0]);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = (v[i][e] - mean) * inv * gm[e];
        if (beta) {
          const float* bt = reinterpret_cast<const float*>(&bt_raw[i][0]);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[i][e] += bt[e];
        }
      }
      *reinterpret_cast<uint4*>(xs + (size_t)r * stride + k) = pack8(v[i]);
    }
    // columns of the staged width that lie beyond the vectors held in registers: zero
    for (int k = (tr + VPT * tpr) * 8; live && k < width; k += tpr * 8)
      *reinterpret_cast<uint4*>(xs + (size_t)r * stride + k) = make_uint4(0u, 0u, 0u, 0u);
  }
}

// Columns [k_lo, k_lo + width) of the M rows of X into shared memory as bf16 (no norm); columns
// at or beyond K are zero.  The vectors are spread over all threads of the block.
template <typename TX>
__device__ __forceinline__ void stage_rows_copy(const TX* X, bf16* xs, int stride,
                                                int M, int K, int k_lo, int width, int tid,
                                                int n_threads) {
  const int vpr = width >> 3;   // vectors per row
  for (int idx = tid; idx < M * vpr; idx += n_threads) {
    const int r = idx / vpr, kk = (idx - r * vpr) * 8, k = k_lo + kk;
    uint4 packed = make_uint4(0u, 0u, 0u, 0u);
    if (k < K) {
      float v[8];
      load8(X + (size_t)r * K + k, v);
      packed = pack8(v);
    }
    *reinterpret_cast<uint4*>(xs + (size_t)r * stride + kk) = packed;
  }
}

// K is cut into segments of `kseg` columns (a multiple of 32 * WARPS) so that the staged rows
// fit in shared memory; within a segment chunk c of 32 columns belongs to warp c % WARPS.
// With a single segment the rows are staged once and the CTA walks over column groups
// blockIdx.x, blockIdx.x + gridDim.x, ... with the next group's weights already in flight.
// Only the M real rows live in shared memory; the other rows of the 16-row MMA tile are zero
// registers.  A fused norm needs a single segment (the launcher sees to it).
template <int MT, int WARPS, typename TX, int VPT, int CH, typename TOut>
__global__ void __launch_bounds__(WARPS * 32, (CH <= 4 && VPT <= 3 && MT == 1) ? 2 : 1)
gemm_skinny_bf16_kernel(const TX* X, const float* __restrict__ gamma,
                        const float* __restrict__ beta, float eps, const bf16* __restrict__ W,
                        const float* __restrict__ bias, const float* residual, TOut* out, int M,
                        int N, int K, int act, int kseg, int tpr) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr bool LN = VPT > 0;   // VPT: vectors of a row per thread for the fused norm; 0 = none
  constexpr int NT = WARPS * 32;
  constexpr int EPT = (MT * 16 * 8 + NT - 1) / NT;   // outputs per thread and column group
  const int stride = kseg + 8;
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);                           // [M][stride]
  float* red = reinterpret_cast<float*>(smem_raw + (((size_t)M * stride * sizeof(bf16) + 15) & ~(size_t)15));
  float* part = red + WARPS * MT * 16 * 8;                                // [WARPS]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n_groups = (N + 7) / 8;
  const int rounds_per_seg = kseg / (32 * WARPS);
  const int n_rounds = (K + 32 * WARPS - 1) / (32 * WARPS);   // round j: chunk j * WARPS + warp
  const bool single = n_rounds <= rounds_per_seg;

  uint4 wreg[CH];
  auto load_batch = [&](int grp_, int j0, int cnt) {
    const int n = grp_ * 8 + g;
    const bf16* wrow = W + (size_t)(n < N ? n : 0) * K;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int k = ((j0 + i) * WARPS + warp) * 32 + t * 8;
      if (i < cnt && k < K && n < N && grp_ < n_groups)
        wreg[i] = __ldg(reinterpret_cast<const uint4*>(wrow + k));
      else
        wreg[i] = make_uint4(0u, 0u, 0u, 0u);
    }
  };
  auto batch_len = [&](int j) {   // rounds from j to the end of j's segment, at most CH
    const int seg_end = min(n_rounds, (j / rounds_per_seg + 1) * rounds_per_seg);
    return max(0, min(CH, seg_end - j));
  };
  int grp = blockIdx.x;
  load_batch(grp, 0, batch_len(0));   // weights: in flight while the predecessor finishes and
                                      // the rows are staged
  nb_grid_dependency_wait();

  // what the epilogue of a column group needs, asked for ahead of time
  float e_bias[EPT], e_res[EPT];
  auto load_epilogue = [&](int grp_) {
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
      const int idx = tid + i * NT;
      const int row = idx >> 3, nn = grp_ * 8 + (idx & 7);
      const bool live = idx < MT * 16 * 8 && row < M && nn < N && grp_ < n_groups;
      e_bias[i] = (live && bias) ? __ldg(bias + nn) : 0.0f;
      e_res[i] = (live && residual) ? residual[(size_t)row * N + nn] : 0.0f;
    }
  };
  load_epilogue(grp);

  if constexpr (LN) {
    stage_rows_norm<NT, (VPT > 0 ? VPT : 1)>(reinterpret_cast<const float*>(X), xs, stride, M, K,
                                             kseg, gamma, beta, eps, part, tid, tpr);
  } else {
    if (single) stage_rows_copy<TX>(X, xs, stride, M, K, 0, kseg, tid, NT);
  }
  if (single) __syncthreads();

  // rows of the MMA tile that exist
  bool row_a[MT], row_b[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    row_a[m] = m * 16 + g < M;
    row_b[m] = m * 16 + g + 8 < M;
  }

  for (; grp < n_groups; grp += gridDim.x) {
    const int n0 = grp * 8;
    float acc[MT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[m][j] = 0.0f;

    for (int seg0 = 0; seg0 < n_rounds; seg0 += rounds_per_seg) {
      const int seg_end = min(n_rounds, seg0 + rounds_per_seg);
      const int k_lo = seg0 * 32 * WARPS;
      if (!single) {
        if (seg0 > 0) __syncthreads();   // everyone is done reading the previous segment
        stage_rows_copy<TX>(X, xs, stride, M, K, k_lo, kseg, tid, NT);
        __syncthreads();
      }
      for (int j = seg0; j < seg_end; j += CH) {
        const int cnt = min(CH, seg_end - j);
#pragma unroll
        for (int i = 0; i < CH; ++i) {
          if (i < cnt) {
            const int kk = ((j + i) * WARPS + warp) * 32 + t * 8 - k_lo;   // column within xs
            const uint4 w = wreg[i];
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              uint4 xa = make_uint4(0u, 0u, 0u, 0u), xb = make_uint4(0u, 0u, 0u, 0u);
              if (row_a[m])
                xa = *reinterpret_cast<const uint4*>(xs + (size_t)(m * 16 + g) * stride + kk);
              if (row_b[m])
                xb = *reinterpret_cast<const uint4*>(xs + (size_t)(m * 16 + g + 8) * stride + kk);
              // K is permuted inside a chunk: lane group t owns elements 8t..8t+7 of both
              // operands
              mma_bf16_16816(acc[m], xa.x, xb.x, xa.y, xb.y, w.x, w.y);
              mma_bf16_16816(acc[m], xa.z, xb.z, xa.w, xb.w, w.z, w.w);
            }
          }
        }
        // the next batch: of this group, or the first of the next group this CTA takes
        if (j + cnt < n_rounds)
          load_batch(grp, j + cnt, batch_len(j + cnt));
        else
          load_batch(grp + gridDim.x, 0, batch_len(0));
      }
    }

    // the next kernel may be set up from here on: this CTA's weights are in, what is left is
    // the reduction and the epilogue (with the trigger at the start of the kernel, or after the
    // rows were staged, the successor's loads fight this kernel's for the memory system and a
    // decode step takes 6 % longer than without any overlap; here it takes 3 % less)
    if (grp + (int)gridDim.x >= n_groups) nb_launch_dependents();
    // partial sums of the warps -> shared memory -> epilogue
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float* r0 = red + ((size_t)warp * MT * 16 + m * 16 + g) * 8 + t * 2;
      float* r1 = r0 + 8 * 8;
      r0[0] = acc[m][0];
      r0[1] = acc[m][1];
      r1[0] = acc[m][2];
      r1[1] = acc[m][3];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
      const int idx = tid + i * NT;
      const int row = idx >> 3, col = idx & 7;
      const int nn = n0 + col;
      if (idx >= MT * 16 * 8 || row >= M || nn >= N) continue;
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) v += red[((size_t)w * MT * 16 + row) * 8 + col];
      v += e_bias[i];
      v = nb_apply_act_fast(v, act);
      v += e_res[i];
      out[(size_t)row * N + nn] = nb_from_f32<TOut>(v);
    }
    load_epilogue(grp + gridDim.x);   // for the next group this CTA takes
    __syncthreads();   // `red` is rewritten for the next group
  }
}

// fp32 weights on the CUDA cores: one warp per output column, lanes along K, rows in chunks
// of 8 held in shared memory.
constexpr int F32_WARPS = 8;
constexpr int F32_ROWS = 8;

template <typename TX, bool LN, typename TOut>
__global__ void __launch_bounds__(F32_WARPS * 32)
gemm_skinny_f32_kernel(const TX* X, const float* __restrict__ gamma,
                       const float* __restrict__ beta, float eps, const float* __restrict__ W,
                       const float* __restrict__ bias, const float* residual, TOut* out, int M,
                       int N, int K, int act) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* xs = reinterpret_cast<float*>(smem_raw);  // [F32_ROWS][K]
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.x * F32_WARPS + warp;
  const float* wrow = W + (size_t)(n < N ? n : 0) * K;
  const bool vec = (K % 4 == 0);

  for (int m0 = 0; m0 < M; m0 += F32_ROWS) {
    const int rows = min(F32_ROWS, M - m0);
    __syncthreads();
    for (int r = warp; r < F32_ROWS; r += F32_WARPS) {
      float* dst = xs + (size_t)r * K;
      if (r >= rows) {
        for (int k = lane; k < K; k += 32) dst[k] = 0.0f;
        continue;
      }
      const TX* src = X + (size_t)(m0 + r) * K;
      if constexpr (LN) {
        float s = 0.0f;
        for (int k = lane; k < K; k += 32) s += nb_to_f32(src[k]);
        const float mean = nb_warp_sum(s) / (float)K;
        float q = 0.0f;
        for (int k = lane; k < K; k += 32) {
          const float c = nb_to_f32(src[k]) - mean;
          q += c * c;
        }
        const float inv = 1.0f / sqrtf(nb_warp_sum(q) / (float)K + eps);
        for (int k = lane; k < K; k += 32) {
          float y = (nb_to_f32(src[k]) - mean) * inv * gamma[k];
          if (beta) y += beta[k];
          dst[k] = y;
        }
      } else {
        for (int k = lane; k < K; k += 32) dst[k] = nb_to_f32(src[k]);
      }
    }
    __syncthreads();
    float acc[F32_ROWS];
#pragma unroll
    for (int r = 0; r < F32_ROWS; ++r) acc[r] = 0.0f;
    if (n < N) {
      if (vec) {
        for (int k = lane * 4; k < K; k += 128) {
          const float4 w = __ldg(reinterpret_cast<const float4*>(wrow + k));
#pragma unroll
          for (int r = 0; r < F32_ROWS; ++r) {
            const float4 x = *reinterpret_cast<const float4*>(xs + (size_t)r * K + k);
            acc[r] = fmaf(x.x, w.x, acc[r]);
            acc[r] = fmaf(x.y, w.y, acc[r]);
            acc[r] = fmaf(x.z, w.z, acc[r]);
            acc[r] = fmaf(x.w, w.w, acc[r]);
          }
        }
      } else {
        for (int k = lane; k < K; k += 32) {
          const float w = __ldg(wrow + k);
#pragma unroll
          for (int r = 0; r < F32_ROWS; ++r) acc[r] = fmaf(xs[(size_t)r * K + k], w, acc[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < F32_ROWS; ++r) acc[r] = nb_warp_sum(acc[r]);
    if (lane == 0 && n < N) {
      for (int r = 0; r < rows; ++r) {
        float v = acc[r];
        if (bias) v += bias[n];
        v = nb_apply_act(v, act);
        const size_t o = (size_t)(m0 + r) * N + n;
        if (residual) v += residual[o];
        out[o] = nb_from_f32<TOut>(v);
      }
    }
  }
}

// Threads that share a row while it is normalised: the block divided by the rows (rounded up
// to a power of two), at least a warp.
inline int norm_threads_per_row(int n_threads, int M) {
  int mp = 1;
  while (mp < M) mp <<= 1;
  return n_threads / mp < 32 ? 32 : n_threads / mp;
}

template <int MT, int WARPS, typename TX, int VPT, int CH, typename TOut>
int launch_bf16_c(const void* X, const float* gamma, const float* beta, float eps, const void* W,
                const float* bias, const float* residual, void* out, int M, int N, int K, int act,
                cudaStream_t stream) {
  // segment of K whose staged rows take about 96 KB at most (two CTAs per SM)
  constexpr int NT = WARPS * 32;
  const int unit = 32 * WARPS;
  const int cap = (96 * 1024) / (M * (int)sizeof(bf16));
  int kseg = ((K + unit - 1) / unit) * unit;
  const bool single = kseg <= cap;
  if (!single) kseg = (cap / unit) * unit;
  if (kseg < unit) kseg = unit;
  constexpr bool LN = VPT > 0;
  const int tpr = norm_threads_per_row(NT, M);
  if (LN) {
    NB_REQUIRE(single && K <= 8 * tpr * VPT, NB_ERR_UNSUPPORTED,
               "gemm_skinny: a fused norm takes rows up to %d wide for %d rows (got %d)",
               8 * tpr * VPT, M, K);
  }
  const size_t xs_bytes = (((size_t)M * (kseg + 8) * sizeof(bf16)) + 15) & ~(size_t)15;
  const size_t smem = xs_bytes + (size_t)WARPS * MT * 16 * 8 * sizeof(float) + WARPS * sizeof(float);
  auto kern = gemm_skinny_bf16_kernel<MT, WARPS, TX, VPT, CH, TOut>;
  if (smem > 48 * 1024)
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int n_groups = (N + 7) / 8;
  static int resident = 0;   // CTAs of this instantiation that fit on the GPU at once
  static size_t resident_smem = 0;
  if (resident == 0 || resident_smem != smem) {
    int per_sm = 0, dev = 0, sms = 0;
    NB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NT, smem));
    NB_CUDA(cudaGetDevice(&dev));
    NB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    resident = (per_sm > 0 ? per_sm : 1) * (sms > 0 ? sms : 1);
    resident_smem = smem;
  }
  // with one segment the rows are staged once per CTA and the CTA walks over column groups
  const int grid = (single && n_groups > resident) ? resident : n_groups;
  NB_CUDA(nb_launch(kern, dim3(grid), dim3(NT), smem, stream, (const TX*)X, gamma, beta, eps,
                    (const bf16*)W, bias, residual, (TOut*)out, M, N, K, act, kseg, tpr));
  return 0;
}

// Picks how many chunks of weights a warp holds at a time.
template <int MT, int WARPS, typename TX, int VPT, typename TOut>
int launch_bf16_v(const void* X, const float* gamma, const float* beta, float eps, const void* W,
                  const float* bias, const float* residual, void* out, int M, int N, int K, int act,
                  cudaStream_t stream) {
  const int n_rounds = (K + 32 * WARPS - 1) / (32 * WARPS);
  if (n_rounds <= 4)
    return launch_bf16_c<MT, WARPS, TX, VPT, 4, TOut>(X, gamma, beta, eps, W, bias, residual, out, M,
                                                      N, K, act, stream);
  return launch_bf16_c<MT, WARPS, TX, VPT, 12, TOut>(X, gamma, beta, eps, W, bias, residual, out, M,
                                                     N, K, act, stream);
}

// Picks the number of row vectors per thread for the fused norm (0 without a norm).
template <int MT, int WARPS, typename TX, bool LN, typename TOut>
int launch_bf16(const void* X, const float* gamma, const float* beta, float eps, const void* W,
                const float* bias, const float* residual, void* out, int M, int N, int K, int act,
                cudaStream_t stream) {
#define NB_V(V_) \
  return launch_bf16_v<MT, WARPS, TX, V_, TOut>(X, gamma, beta, eps, W, bias, residual, out, M, N, K, act, stream)
  if constexpr (!LN) {
    NB_V(0);
  } else {
    const int tpr = norm_threads_per_row(WARPS * 32, M);
    const int vpt = (K / 8 + tpr - 1) / tpr;
    if (vpt <= 1) NB_V(1);
    if (vpt <= 2) NB_V(2);
    if (vpt <= 3) NB_V(3);
    if (vpt <= 4) NB_V(4);
    NB_V(8);
  }
#undef NB_V
}

template <typename TX, bool LN, typename TOut>
int dispatch_bf16(const void* X, const float* gamma, const float* beta, float eps, const void* W,
                  const float* bias, const float* residual, void* out, int M, int N, int K,
                  int act, cudaStream_t stream) {
  const bool wide = K > 1024;
#define NB_GO(MT_, W_) \
  return launch_bf16<MT_, W_, TX, LN, TOut>(X, gamma, beta, eps, W, bias, residual, out, M, N, K, act, stream)
  // eight warps when K is long, or when a fused norm has more than four rows to bring in
  if (M <= 16) { if (wide || (LN && M > 4)) NB_GO(1, 8); else NB_GO(1, 4); }
  if constexpr (LN) {
    NB_REQUIRE(false, NB_ERR_UNSUPPORTED,
               "gemm_skinny: the fused norm takes at most 16 rows (got %d)", M);
  } else {
    if (M <= 32) { if (wide) NB_GO(2, 8); else NB_GO(2, 4); }
    if (wide) NB_GO(4, 8); else NB_GO(4, 4);
  }
#undef NB_GO
}

template <typename TX, bool LN, typename TOut>
int launch_f32(const void* X, const float* gamma, const float* beta, float eps, const void* W,
               const float* bias, const float* residual, void* out, int M, int N, int K, int act,
               cudaStream_t stream) {
  const size_t smem = (size_t)F32_ROWS * K * sizeof(float);
  NB_REQUIRE(smem <= 220 * 1024, NB_ERR_UNSUPPORTED,
             "gemm_skinny: width %d needs %zu bytes of shared memory", K, smem);
  auto kern = gemm_skinny_f32_kernel<TX, LN, TOut>;
  if (smem > 48 * 1024)
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  NB_CUDA(nb_launch(kern, dim3((N + F32_WARPS - 1) / F32_WARPS), dim3(F32_WARPS * 32), smem, stream,
                    (const TX*)X, gamma, beta, eps, (const float*)W, bias, residual, (TOut*)out, M,
                    N, K, act));
  return 0;
}

}  // namespace

// Whether nb_gemm_skinny can apply the LayerNorm of the rows itself (bf16 weights): at most 16
// rows that fit in shared memory in one piece and are short enough for the registers of the
// threads that share a row.  Else the caller normalises the rows first.
NB_EXPORT int nb_gemm_skinny_norm_supported(int M, int N, int K) {
  if (M < 1 || M > 16 || N < 1 || K < 8 || K % 8) return 0;
  const int warps = (K > 1024 || M > 4) ? 8 : 4;   // as dispatch_bf16 picks them
  const int unit = 32 * warps;
  const int kseg = ((K + unit - 1) / unit) * unit;
  if (kseg > (96 * 1024) / (M * (int)sizeof(bf16))) return 0;
  return K <= 8 * norm_threads_per_row(warps * 32, M) * 8;
}

// M <= 64.  gamma != nullptr asks for LayerNorm of the rows first (X must then be fp32).
// bf16 weights need K % 8 == 0 and 16-byte aligned rows; `residual` may alias `out` (fp32).
NB_EXPORT int nb_gemm_skinny(const void* X, int x_dtype, const float* gamma, const float* beta,
                             float eps, const void* W, int w_dtype, const float* bias,
                             const float* residual, void* out, int out_dtype, int M, int N, int K,
                             int act, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  NB_REQUIRE(M > 0 && M <= 64 && N > 0 && K > 0, NB_ERR_UNSUPPORTED,
             "gemm_skinny: takes 1..64 rows, got M=%d N=%d K=%d", M, N, K);
  const bool ln = gamma != nullptr;
  NB_REQUIRE(!ln || x_dtype == NB_F32, NB_ERR_BAD_ARG, "gemm_skinny: a fused norm needs fp32 rows");
  int rc = 0;
#define NB_OUT(FN, TX_, LN_)                                                                  \
  rc = (out_dtype == NB_F32)                                                                  \
           ? FN<TX_, LN_, float>(X, gamma, beta, eps, W, bias, residual, out, M, N, K, act, stream) \
           : FN<TX_, LN_, bf16>(X, gamma, beta, eps, W, bias, residual, out, M, N, K, act, stream)
  if (w_dtype == NB_BF16) {
    NB_REQUIRE(K % 8 == 0 && (uintptr_t)W % 16 == 0, NB_ERR_UNSUPPORTED,
               "gemm_skinny: bf16 weights need a width that is a multiple of 8 (got %d)", K);
    NB_REQUIRE((uintptr_t)X % 16 == 0 && (uintptr_t)gamma % 16 == 0 && (uintptr_t)beta % 16 == 0,
               NB_ERR_UNSUPPORTED, "gemm_skinny: rows and norm vectors must be 16-byte aligned");
    if (x_dtype == NB_F32) { if (ln) { NB_OUT(dispatch_bf16, float, true); } else { NB_OUT(dispatch_bf16, float, false); } }
    else { NB_OUT(dispatch_bf16, bf16, false); }
  } else {
    NB_REQUIRE((uintptr_t)W % 16 == 0, NB_ERR_UNSUPPORTED, "gemm_skinny: unaligned weights");
    if (x_dtype == NB_F32) { if (ln) { NB_OUT(launch_f32, float, true); } else { NB_OUT(launch_f32, float, false); } }
    else { NB_OUT(launch_f32, bf16, false); }
  }
#undef NB_OUT
  if (rc) return rc;
  NB_CHECK_LAUNCH("gemm_skinny");
  return 0;
}
