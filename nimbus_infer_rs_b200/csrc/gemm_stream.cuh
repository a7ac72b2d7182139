// The kernel, the plan and the launchers of the decode step's matrix product (see
// gemm_stream.cu for what it does).  Two translation units include this file, one for each
// type of the result, so that the many instantiations of the kernel compile side by side;
// only gemm_stream.cu plans a product, the other unit is handed the plan.
#pragma once
#include "tc05_common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void load8f(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8f(const bf16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __bfloat162float(h[i].x);
    v[2 * i + 1] = __bfloat162float(h[i].y);
  }
}
__device__ __forceinline__ uint4 pack8f(const float (&v)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return u;
}

// Sum over the `tpr` consecutive threads that share a row (a power of two; a multiple of 32
// goes through `part`, one float per warp).  Every thread of the block calls it.
__device__ __forceinline__ float row_sum(float v, float* part, int tid, int tpr) {
  if (tpr <= 32) {
    for (int o = tpr >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
  }
  v = nb_warp_sum(v);
  __syncthreads();
  if ((tid & 31) == 0) part[tid >> 5] = v;
  __syncthreads();
  const int first = (tid / tpr) * (tpr >> 5);
  float s = 0.0f;
  for (int w = 0; w < (tpr >> 5); ++w) s += part[first + w];
  return s;
}


struct StreamShape {
  int GB;         // groups of 16 columns per batch (a power of two)
  int wn;         // warps side by side along the columns (the others split K)
  int n_kbox;     // 64-column boxes of K per work item
  int n_kc;       // work items per batch
  int S;          // stages of the ring
  int x_stride;   // elements between staged rows
  int tpr;        // threads that share a row while it is normalised
  int n16;        // groups of 16 columns of the whole product
  unsigned vpr_magic;   // ceil(2^32 / vectors per staged row): index / vectors = umulhi(index, magic)
};

// The tensor-core instruction takes 16 x 16 of one operand and 16 x 8 of the other.  The weights
// are the 16-row operand (16 output columns), the step's rows the 8-wide one: with at most 8
// rows nothing of an instruction is wasted; rows 9..16 (HI) take a second instruction.
//
// Weights come as TMA boxes of (rows of a batch) x 64 columns, 128-byte swizzled: a row of a
// box is 128 bytes, and its 16-byte pieces are stored at (piece ^ (row & 7)), so the eight
// rows a quarter warp reads lie in eight different bank groups.  Rows beyond N and columns
// beyond K arrive as zeros.
//
// NW warps; GPW: column groups a warp takes per batch (GB = wn * GPW); VPT: 8-element vectors
// of a row a thread holds while the row is normalised (0: no norm).
template <int NW, int GPW, typename TX, int VPT, bool HI, typename TOut>
__global__ void __launch_bounds__(NW * 32)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const TX* X,
                   const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                   const float* __restrict__ bias, const float* residual, TOut* out, int M, int N,
                   int K, int act, StreamShape sh, int* err_word) {
  constexpr bool LN = VPT > 0;
  constexpr int NT = NW * 32;
  constexpr int NH = HI ? 2 : 1;
  constexpr int MP = HI ? 16 : 8;          // rows of the step as the instruction sees them
  // 32-column steps per turn of the product loop (four, with eight accumulators, measured
  // slower: 0.392 against 0.354 ms a decode step at batch 8)
  constexpr int SPI = 2;
  constexpr int NCH = 2 * SPI;             // accumulators per column group and half
  constexpr int EPT = 4;                   // outputs a thread finishes per batch when warps split K
  constexpr int ROUND = sizeof(TX) == 2 ? 12 : 6;   // vectors a thread copies per trip to L2
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;              // swizzle atoms are 1024 bytes
  unsigned char* smem = smem_dyn + (base - raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rows_b = sh.GB * 16;                             // weight rows (= output columns) of a batch
  const int box_bytes = rows_b * 128;
  const int stage_bytes = sh.n_kbox * box_bytes;
  const int k_pad = ((K + 31) / 32) * 32;
  const int n_box_k = (K + 63) >> 6;                         // boxes along K of the whole matrix
  const int wk = NW / sh.wn;                                 // warps that split K
  // layout: [S stages of weights][M staged rows][partial sums][norm weight, bias][barriers]
  unsigned char* w_s = smem;
  bf16* x_s = reinterpret_cast<bf16*>(smem + (size_t)sh.S * stage_bytes);
  float* red = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(x_s) +
                                        (((size_t)M * sh.x_stride * sizeof(bf16) + 15) & ~(size_t)15));
  float* gb_s = red + (wk > 1 ? wk * MP * rows_b : 0);       // [2][k_pad] when LN
  float* part = gb_s + (LN ? 2 * k_pad : 0);                 // [NW]
  uint64_t* bars = reinterpret_cast<uint64_t*>(part + NW);   // [S]; NW is even
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + sh.S);
  const uint32_t bars32 = smem_u32(bars);

  // this CTA's column groups: an even share of the product's, in one run
  const int grp_lo = (int)(((long long)blockIdx.x * sh.n16) / gridDim.x);
  const int grp_hi = (int)(((long long)(blockIdx.x + 1) * sh.n16) / gridDim.x);
  const int n_batches = (grp_hi - grp_lo + sh.GB - 1) / sh.GB;
  const int n_items = n_batches * sh.n_kc;

  // work item -> its boxes.  Called by every lane of warp 0 with the item's batch and chunk.
  auto issue = [&](int s, int bi, int c) {
    const int n0 = (grp_lo + bi * sh.GB) * 16;
    const int box0 = c * sh.n_kbox;
    const int nb = min(sh.n_kbox, n_box_k - box0);
    const uint32_t bar = bars32 + 8u * s;
    if (lane == 0) mbar_expect_tx(bar, (uint32_t)(nb * box_bytes));
    __syncwarp();
    for (int j = lane; j < nb; j += 32)
      tma_load_2d(base + (uint32_t)(s * stage_bytes + j * box_bytes), &map_w, (box0 + j) * 64, n0, bar);
  };

  if (tid == 0) {
    for (int s = 0; s < sh.S; ++s) mbar_init(bars32 + 8u * s, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  __syncthreads();
  int fill_item = 0, fill_s = 0, fill_b = 0, fill_c = 0;   // the next item to ask for (warp 0)
  if (warp == 0) {
    const int first = min(n_items, sh.S);
    for (; fill_item < first; ++fill_item) {
      issue(fill_s, fill_b, fill_c);
      if (++fill_s == sh.S) fill_s = 0;
      if (++fill_c == sh.n_kc) { fill_c = 0; ++fill_b; }
    }
  }

  // ---- constants, indices and addresses, while the kernel in front finishes: after the wait
  // every instruction is on the step's critical path
  if constexpr (LN) {   // the norm's weight and bias, zero beyond K
    for (int k = tid; k < k_pad; k += NT) {
      gb_s[k] = k < K ? __ldg(gamma + k) : 0.0f;
      gb_s[k_pad + k] = (k < K && beta != nullptr) ? __ldg(beta + k) : 0.0f;
    }
  }
  const int gw = warp % sh.wn, kpart = warp / sh.wn;
  // when warps split K, thread `tid` finishes outputs e = tid, tid + NT, ... of a batch:
  // row e / rows_b of the step, column e % rows_b of the batch (rows_b is a power of two)
  const int rb_shift = 31 - __clz(rows_b);
  float e_bias[EPT];
  int e_off[EPT];          // where the output lies (first batch), -1: none
#pragma unroll
  for (int j = 0; j < EPT; ++j) {
    const int e = tid + j * NT;
    const int m = e >> rb_shift, n = grp_lo * 16 + (e & (rows_b - 1));
    const bool live = wk > 1 && m < M && n < N && n < grp_hi * 16;
    e_off[j] = live ? m * N + n : -1;
    e_bias[j] = (live && bias != nullptr) ? __ldg(bias + n) : 0.0f;
  }
  // the instruction's operands in shared memory
  const bool row_lo = g < M, row_hi = HI && (g + 8 < M);
  const bf16* x_lo = x_s + (size_t)g * sh.x_stride + t * 8;
  const bf16* x_hi = x_s + (size_t)(g + 8) * sh.x_stride + t * 8;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  // byte offsets of this lane's two pieces in a row of a box (even and odd 32-column step)
  const int piece0 = ((t ^ g) & 7) << 4, piece1 = (((4 + t) ^ g) & 7) << 4;
  const int w_row0 = (gw * 16 + g) * 128;                  // row g of the warp's first group
  // accumulators: one per instruction of a turn (see the loop)
  float acc[GPW][NH][NCH][4];
#pragma unroll
  for (int i = 0; i < GPW; ++i)
#pragma unroll
    for (int h = 0; h < NH; ++h)
#pragma unroll
      for (int q = 0; q < NCH; ++q)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][h][q][j] = 0.0f;
  // staging: which vectors this thread brings in
  [[maybe_unused]] int st_src[ROUND], st_dst[ROUND];
  [[maybe_unused]] const int vpr = k_pad >> 3;
  [[maybe_unused]] const int total = M * vpr;
  if constexpr (!LN) {
#pragma unroll
    for (int j = 0; j < ROUND; ++j) {
      const int idx = tid + j * NT;
      const int r = (int)__umulhi((unsigned)idx, sh.vpr_magic);
      const int k = (idx - r * vpr) * 8;
      st_dst[j] = idx < total ? r * sh.x_stride + k : -1;
      st_src[j] = (idx < total && k < K) ? r * K + k : -1;
    }
  }
  [[maybe_unused]] const int ln_rpp = NT / sh.tpr;         // rows normalised per pass
  [[maybe_unused]] const int ln_tr = tid % sh.tpr, ln_row = tid / sh.tpr;
  const float inv_k = 1.0f / (float)K;

  nb_grid_dependency_wait();
  // this kernel's weights were asked for long ago: the kernel behind it may start and ask for
  // its own (only now: see common.cuh on what a kernel may read before its wait)
  nb_launch_dependents();

  // what the first batch's epilogue adds, asked for before anything else
  float e_res[EPT];
#pragma unroll
  for (int j = 0; j < EPT; ++j)
    e_res[j] = (residual != nullptr && e_off[j] >= 0) ? residual[e_off[j]] : 0.0f;

  // ---- stage the rows (the only data of the step this kernel reads)
  if constexpr (LN) {
    const float* Xf = reinterpret_cast<const float*>(X);
    for (int r0 = 0; r0 < M; r0 += ln_rpp) {
      const int r = r0 + ln_row;
      const bool live = r < M;
      const float* src = Xf + (size_t)(live ? r : 0) * K;
      float v[VPT][8];
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int k = (ln_tr + i * sh.tpr) * 8;
        if (live && k < K) {
          load8f(src + k, v[i]);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[i][e] = 0.0f;
        }
      }
      // mean, then the variance of the centred values (two passes over the registers,
      // src/ops.rs:32-40), each summed in a small tree
      float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) s4[e & 3] += v[i][e];
      const float mean = row_sum((s4[0] + s4[1]) + (s4[2] + s4[3]), part, tid, sh.tpr) * inv_k;
      float q4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        if (live && (ln_tr + i * sh.tpr) * 8 < K) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float c = v[i][e] - mean;
            q4[e & 3] = fmaf(c, c, q4[e & 3]);
          }
        }
      }
      const float var = row_sum((q4[0] + q4[1]) + (q4[2] + q4[3]), part, tid, sh.tpr) * inv_k;
      const float inv = rsqrtf(var + eps);
      if (r0 == 0) __syncthreads();   // gb_s is complete (written before the wait by all threads)
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int k = (ln_tr + i * sh.tpr) * 8;
        if (!live || k >= k_pad) continue;
        if (k < K) {
          float gm[8], bt[8];
          load8f(gb_s + k, gm);
          load8f(gb_s + k_pad + k, bt);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[i][e] = fmaf((v[i][e] - mean) * inv, gm[e], bt[e]);
        }
        *reinterpret_cast<uint4*>(x_s + (size_t)r * sh.x_stride + k) = pack8f(v[i]);
      }
    }
  } else {
    // vectors of 8 columns, all threads side by side; the loads of a round are all asked for
    // before the first is used (one trip to L2 per round)
    for (int base_idx = tid; base_idx < total; base_idx += ROUND * NT) {
      float v[ROUND][sizeof(TX) == 2 ? 1 : 8];
      uint4 rawv[ROUND];
      if (base_idx != tid) {   // a later round: its indices
#pragma unroll
        for (int j = 0; j < ROUND; ++j) {
          const int idx = base_idx + j * NT;
          const int r = (int)__umulhi((unsigned)idx, sh.vpr_magic);
          const int k = (idx - r * vpr) * 8;
          st_dst[j] = idx < total ? r * sh.x_stride + k : -1;
          st_src[j] = (idx < total && k < K) ? r * K + k : -1;
        }
      }
#pragma unroll
      for (int j = 0; j < ROUND; ++j) {
        rawv[j] = zero4;
        if constexpr (sizeof(TX) == 2) {
          if (st_src[j] >= 0) rawv[j] = *reinterpret_cast<const uint4*>(X + st_src[j]);
        } else {
          if (st_src[j] >= 0) {
            load8f(X + st_src[j], v[j]);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[j][e] = 0.0f;
          }
        }
      }
#pragma unroll
      for (int j = 0; j < ROUND; ++j) {
        if (st_dst[j] < 0) continue;
        if constexpr (sizeof(TX) != 2) rawv[j] = pack8f(v[j]);
        *reinterpret_cast<uint4*>(x_s + st_dst[j]) = rawv[j];
      }
    }
  }
  __syncthreads();

  // ---- the walk over work items
  bool ok = true;
  int bi = 0, c = 0;                      // batch and chunk of the item
  int s = 0;                              // its stage, and the phase of that stage's barrier
  uint32_t phase = 0;
  for (int item = 0; item < n_items; ++item) {
    const int grp0 = grp_lo + bi * sh.GB;
    if (ok) ok = mbar_wait(bars32 + 8u * s, phase, abort_flag);
    const unsigned char* st = w_s + (size_t)s * stage_bytes + w_row0;
    if (ok) {
      const int k0 = c * sh.n_kbox * 64;
      const int steps = min(sh.n_kbox * 2, (k_pad - k0) >> 5);       // 32-column steps of the item
      for (int ks = kpart; ks < steps; ks += SPI * wk) {
        // SPI 32-column steps per turn, two instructions each, every one with an accumulator
        // of its own: a tensor-core instruction of this kind takes a few hundred clocks to hand
        // its result on, so none of a turn's instructions waits for another
        uint4 xl[SPI], xh[SPI], wa[GPW][SPI], wb[GPW][SPI];
#pragma unroll
        for (int u = 0; u < SPI; ++u) {
          const int k1 = ks + u * wk;
          const bool in = k1 < steps;
          xl[u] = (row_lo && in) ? *reinterpret_cast<const uint4*>(x_lo + k0 + k1 * 32) : zero4;
          xh[u] = (row_hi && in) ? *reinterpret_cast<const uint4*>(x_hi + k0 + k1 * 32) : zero4;
          const int off = (k1 >> 1) * box_bytes + ((k1 & 1) ? piece1 : piece0);
#pragma unroll
          for (int i = 0; i < GPW; ++i) {
            const unsigned char* wr = st + i * sh.wn * (16 * 128);
            wa[i][u] = in ? *reinterpret_cast<const uint4*>(wr + off) : zero4;
            wb[i][u] = in ? *reinterpret_cast<const uint4*>(wr + 8 * 128 + off) : zero4;
          }
        }
#pragma unroll
        for (int u = 0; u < SPI; ++u) {
#pragma unroll
          for (int i = 0; i < GPW; ++i) {
            // K is permuted inside a 32-column step: lane group t owns columns 8t..8t+7 of both
            // operands, which a dot product does not mind
            mma_16816(acc[i][0][2 * u], wa[i][u].x, wb[i][u].x, wa[i][u].y, wb[i][u].y, xl[u].x, xl[u].y);
            mma_16816(acc[i][0][2 * u + 1], wa[i][u].z, wb[i][u].z, wa[i][u].w, wb[i][u].w, xl[u].z, xl[u].w);
            if constexpr (HI) {
              mma_16816(acc[i][1][2 * u], wa[i][u].x, wb[i][u].x, wa[i][u].y, wb[i][u].y, xh[u].x, xh[u].y);
              mma_16816(acc[i][1][2 * u + 1], wa[i][u].z, wb[i][u].z, wa[i][u].w, wb[i][u].w, xh[u].z, xh[u].w);
            }
          }
        }
      }
    }
    if (++s == sh.S) { s = 0; phase ^= 1u; }
    const bool last_chunk = c == sh.n_kc - 1;
    const bool refill = item + sh.S < n_items;
    if (last_chunk) {
#pragma unroll
      for (int i = 0; i < GPW; ++i)
#pragma unroll
        for (int h = 0; h < NH; ++h)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float a = (acc[i][h][0][j] + acc[i][h][1][j]) + (acc[i][h][2][j] + acc[i][h][3][j]);
            if constexpr (NCH == 8)
              a += (acc[i][h][4][j] + acc[i][h][5][j]) + (acc[i][h][6][j] + acc[i][h][7][j]);
            acc[i][h][0][j] = a;
          }
    }
    // a thread holds, per column group and half: columns g and g + 8 of the group (j = 0,1 and
    // j = 2,3), rows 2t and 2t + 1 of the step (+ 8 in the upper half)
    if (last_chunk && wk > 1) {
      // partial sums of the warps that split K: red[kpart][row of the step][column of the batch]
#pragma unroll
      for (int i = 0; i < GPW; ++i)
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          const int col = (gw + i * sh.wn) * 16 + g;
          float* r0 = red + ((size_t)(kpart * MP + h * 8 + 2 * t) << rb_shift) + col;
          r0[0] = acc[i][h][0][0];
          r0[rows_b] = acc[i][h][0][1];
          r0[8] = acc[i][h][0][2];
          r0[rows_b + 8] = acc[i][h][0][3];
        }
    }
    if (refill || (last_chunk && wk > 1)) __syncthreads();   // stage read by all; sums written
    if (refill && warp == 0) {
      issue(fill_s, fill_b, fill_c);
      if (++fill_s == sh.S) fill_s = 0;
      if (++fill_c == sh.n_kc) { fill_c = 0; ++fill_b; }
    }
    if (++c == sh.n_kc) { c = 0; ++bi; }
    if (!last_chunk) continue;
    // ---- epilogue of the batch
    const int n0 = grp0 * 16;
    const int n_lim = min(N, grp_hi * 16);            // this CTA's columns end here
    if (wk > 1) {
      const bool first = grp0 == grp_lo;
#pragma unroll
      for (int j = 0; j < EPT; ++j) {
        const int e = tid + j * NT;
        const int m = e >> rb_shift, col = e & (rows_b - 1);
        const int n = n0 + col;
        if (m >= M || n >= n_lim || !ok) continue;
        const float* rp = red + ((size_t)m << rb_shift) + col;
        const int pstride = MP << rb_shift;
        float v = 0.0f;
        if (wk == 8) {
          v = ((rp[0] + rp[pstride]) + (rp[2 * pstride] + rp[3 * pstride])) +
              ((rp[4 * pstride] + rp[5 * pstride]) + (rp[6 * pstride] + rp[7 * pstride]));
        } else if (wk == 4) {
          v = (rp[0] + rp[pstride]) + (rp[2 * pstride] + rp[3 * pstride]);
        } else {
          for (int p = 0; p < wk; ++p) v += rp[p * pstride];
        }
        const size_t o = (size_t)m * N + n;
        if (first) {
          v += e_bias[j];
          v = nb_apply_act_fast(v, act);
          v += e_res[j];
        } else {
          if (bias) v += __ldg(bias + n);
          v = nb_apply_act_fast(v, act);
          if (residual) v += residual[o];
        }
        out[o] = nb_from_f32<TOut>(v);
      }
      if (item + 1 < n_items) __syncthreads();   // `red` is written again by the next batch
    } else if (ok) {
#pragma unroll
      for (int i = 0; i < GPW; ++i) {
#pragma unroll
        for (int h = 0; h < NH; ++h) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int n = n0 + (gw + i * sh.wn) * 16 + g + (j >> 1) * 8;
            const int m = h * 8 + 2 * t + (j & 1);
            if (m >= M || n >= n_lim) continue;
            float v = acc[i][h][0][j];
            if (bias) v += __ldg(bias + n);
            v = nb_apply_act_fast(v, act);
            const size_t o = (size_t)m * N + n;
            if (residual) v += residual[o];
            out[o] = nb_from_f32<TOut>(v);
          }
        }
      }
    }
    if (item + 1 < n_items) {   // the next batch starts from zero
#pragma unroll
      for (int i = 0; i < GPW; ++i)
#pragma unroll
        for (int h = 0; h < NH; ++h)
#pragma unroll
          for (int q = 0; q < NCH; ++q)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][h][q][j] = 0.0f;
    }
  }

  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) {
      nb_report_timeout(err_word);
      // let copies that are still in flight land before the shared memory goes away
      const long long t0 = clock64();
      while (clock64() - t0 < 4000000LL) {
      }
    }
    __syncthreads();
  }
}

constexpr int SMEM_LIMIT = 220 * 1024;

// Bytes between rows of `row_bytes` in shared memory such that eight consecutive rows start
// in eight different 16-byte columns of the banks, four apart (16-byte loads of four lanes a
// row, two rows a quarter warp, then run without conflicts).
inline int padded_stride(int row_bytes) {
  int units = (row_bytes + 15) / 16;
  while (units % 8 != 4) ++units;
  return units * 16;
}

struct StreamPlan {
  StreamShape sh;
  int nw;        // warps
  int vpt;       // vectors of a row per thread for the norm (0 without)
  int grid;
  size_t smem;
  bool ok;
};

int g_target_ctas = 0;    // 0: about two CTAs per SM at most; see plan_stream
int g_sms = 0;
int sm_count() {
  if (g_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_sms <= 0)
      g_sms = 148;
  }
  return g_sms;
}

// How a product is cut: see the head of the file.
StreamPlan plan_stream(int M, int N, int K, bool ln) {
  StreamPlan p = {};
  p.ok = false;
  if (M < 1 || M > 16 || N < 1 || K < 8 || K % 8) return p;
  const int sms = sm_count();
  const int n16 = (N + 15) / 16;
  const int k_pad = ((K + 31) / 32) * 32;
  const int n_box_k = (K + 63) / 64;
  // a long walk over many batches per CTA (the output head): every warp takes column groups
  // of its own with K whole, so a batch needs no meeting of partial sums
  const bool walk = n16 > 8 * sms;
  // eight warps when a norm has more than four rows to bring in at once, or K is long
  p.nw = (walk || (ln && M > 4) || K > 1024) ? 8 : 4;
  const int nt = p.nw * 32;
  StreamShape& sh = p.sh;
  sh.n16 = n16;
  sh.vpr_magic = (unsigned)((0x100000000ull + (unsigned)(k_pad / 8) - 1) / (unsigned)(k_pad / 8));
  if ((long long)(M + 16) * (k_pad / 8) >= (1 << 20)) return p;   // the division by multiplication is exact below
  if ((long long)M * N >= (1ll << 31) || (long long)M * K >= (1ll << 31)) return p;   // 32-bit offsets
  int mp = 1;
  while (mp < M) mp <<= 1;
  sh.tpr = nt / mp;
  if (sh.tpr < 8) sh.tpr = 8;
  p.vpt = 0;
  if (ln) {
    int vpt = (k_pad / 8 + sh.tpr - 1) / sh.tpr;
    if (vpt > 4 && sh.tpr < 32) {   // rather two passes over the rows than many registers
      sh.tpr = 32;
      vpt = (k_pad / 8 + sh.tpr - 1) / sh.tpr;
    }
    p.vpt = vpt <= 1 ? 1 : (vpt <= 2 ? 2 : (vpt <= 4 ? 4 : (vpt <= 8 ? 8 : 0)));
    if (p.vpt == 0) return p;   // rows too long for the registers of the threads that share one
  }
  sh.x_stride = padded_stride(k_pad * 2) / 2;
  const size_t x_bytes = (((size_t)M * sh.x_stride * 2) + 15) & ~(size_t)15;
  const size_t tail = (ln ? (size_t)2 * k_pad * 4 : 0) + (size_t)p.nw * 4 + 8 * 8 + 16 + 1024 /* alignment */;
  const int mp_rows = M > 8 ? 16 : 8;
  // CTAs: one per SM for a walk.  Else every CTA gets the same number of column groups (the
  // slowest CTA sets the time), as few as keep the CTAs within one per SM; every CTA stages
  // all the rows, which costs a trip to L2 whatever their number, and the tensor-core
  // instructions of this path are slow, so the work is spread over the SMs.  First choice:
  // whole rows of a CTA's groups in shared memory, everything asked for before the wait; if
  // that does not fit, fewer groups per CTA (more CTAs than SMs then, up to two per SM); if
  // nothing fits whole, K in chunks through a ring of two stages.
  const int cap = (!walk && g_target_ctas > 0) ? g_target_ctas : sms;
  const int per0 = walk ? 0 : (n16 + cap - 1) / cap;
  // (pass 0: whole rows, all CTAs on the GPU at once; pass 1: a ring; pass 2: whole rows, a few
  // CTAs in a second wave)
  for (int pass = 0; pass < (walk ? 1 : 3); ++pass) {
    for (int per = per0; per >= (walk ? 0 : 1); --per) {
      const int ctas = walk ? sms : (n16 + per - 1) / per;
      if (!walk && ctas > 2 * sms) break;
      int GB = 1;
      if (walk) {
        GB = p.nw;
      } else {
        while (GB < per) GB <<= 1;
        if (GB > 2 * p.nw) break;
      }
      for (; GB >= 1; GB >>= 1) {
        if (!walk && GB < per) break;
        sh.GB = GB;
        sh.wn = GB < p.nw ? GB : p.nw;
        const int wk = p.nw / sh.wn;
        if (wk > 1 && (GB * 16 * mp_rows + nt - 1) / nt > 4) continue;   // the epilogue's four outputs a thread
        const size_t red_bytes = wk > 1 ? (size_t)wk * mp_rows * GB * 16 * 4 : 0;
        if (x_bytes + red_bytes + tail >= (size_t)SMEM_LIMIT) continue;
        const size_t room = SMEM_LIMIT - x_bytes - red_bytes - tail;
        const size_t box = (size_t)GB * 16 * 128;
        sh.S = 0;
        if (!walk && pass != 1) {   // whole rows, one item
          if ((size_t)n_box_k * box <= room) {
            sh.n_kbox = n_box_k;
            sh.n_kc = 1;
            sh.S = 1;
          }
        } else {       // a ring: three stages of at most 48 KB for a walk, two large ones else
          const int want = walk ? 3 : 2;
          for (int nkb = n_box_k; nkb >= 1; --nkb) {
            const size_t stage = (size_t)nkb * box;
            const int fit = (int)(room / stage);
            if (!walk && stage < 16 * 1024) break;   // a ring of crumbs: leave it to the other kernel
            if (fit >= want && (!walk || stage <= 48 * 1024 || nkb == 1)) {
              sh.n_kbox = nkb;
              sh.n_kc = (n_box_k + nkb - 1) / nkb;
              sh.S = walk ? (fit < 6 ? fit : 6) : 2;
              if (sh.S > sh.n_kc) sh.S = sh.n_kc;
              break;
            }
          }
        }
        if (sh.S == 0) continue;
        p.smem = (size_t)sh.S * sh.n_kbox * box + x_bytes + red_bytes + tail;
        if (pass == 0 && !walk && ctas > sms && p.smem > (size_t)SMEM_LIMIT / 2) continue;
        p.grid = ctas;
        p.ok = true;
        return p;
      }
      if (walk || pass == 1) break;   // the ring is tried for the widest cut only
    }
  }
  return p;
}

int* error_word() {
  int* w = nb_error_words();
  return w ? w + NB_ERRW_GEMM_STREAM : nullptr;
}

template <int NW, int GPW, typename TX, int VPT, bool HI, typename TOut>
int launch_one(const StreamPlan& p, const void* X, const float* gamma, const float* beta, float eps,
               const void* W, const float* bias, const float* residual, void* out, int M, int N,
               int K, int act, cudaStream_t stream) {
  auto kern = gemm_stream_kernel<NW, GPW, TX, VPT, HI, TOut>;
  static bool configured = false;   // per instantiation
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT));
    configured = true;
  }
  CUtensorMap mw;   // boxes of (rows of a batch) x 64 columns
  const int rc = make_map(&mw, W, N, K, p.sh.GB * 16, 64, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2);
  if (rc) return rc;
  NB_CUDA(nb_launch(kern, dim3(p.grid), dim3(NW * 32), p.smem, stream, mw, (const TX*)X, gamma, beta, eps,
                    bias, residual, (TOut*)out, M, N, K, act, p.sh, error_word()));
  return 0;
}

template <int NW, int GPW, typename TX, int VPT, typename TOut>
int launch_hi(const StreamPlan& p, const void* X, const float* gamma, const float* beta, float eps,
              const void* W, const float* bias, const float* residual, void* out, int M, int N,
              int K, int act, cudaStream_t stream) {
  if (M > 8)
    return launch_one<NW, GPW, TX, VPT, true, TOut>(p, X, gamma, beta, eps, W, bias, residual, out, M, N, K, act, stream);
  return launch_one<NW, GPW, TX, VPT, false, TOut>(p, X, gamma, beta, eps, W, bias, residual, out, M, N, K, act, stream);
}

template <int NW, typename TX, int VPT, typename TOut>
int launch_gpw(const StreamPlan& p, const void* X, const float* gamma, const float* beta, float eps,
               const void* W, const float* bias, const float* residual, void* out, int M, int N,
               int K, int act, cudaStream_t stream) {
  if (p.sh.GB / p.sh.wn == 2)
    return launch_hi<NW, 2, TX, VPT, TOut>(p, X, gamma, beta, eps, W, bias, residual, out, M, N, K, act, stream);
  return launch_hi<NW, 1, TX, VPT, TOut>(p, X, gamma, beta, eps, W, bias, residual, out, M, N, K, act, stream);
}

template <typename TX, int VPT, typename TOut>
int launch_nw(const StreamPlan& p, const void* X, const float* gamma, const float* beta, float eps,
              const void* W, const float* bias, const float* residual, void* out, int M, int N,
              int K, int act, cudaStream_t stream) {
  if (p.nw == 8)
    return launch_gpw<8, TX, VPT, TOut>(p, X, gamma, beta, eps, W, bias, residual, out, M, N, K, act, stream);
  return launch_gpw<4, TX, VPT, TOut>(p, X, gamma, beta, eps, W, bias, residual, out, M, N, K, act, stream);
}

template <typename TX, bool LN, typename TOut>
int launch_vpt(const StreamPlan& p, const void* X, const float* gamma, const float* beta, float eps,
               const void* W, const float* bias, const float* residual, void* out, int M, int N,
               int K, int act, cudaStream_t stream) {
#define NB_V(V_) \
  return launch_nw<TX, V_, TOut>(p, X, gamma, beta, eps, W, bias, residual, out, M, N, K, act, stream)
  if constexpr (!LN) {
    NB_V(0);
  } else {
    if (p.vpt == 1) NB_V(1);
    if (p.vpt == 2) NB_V(2);
    if (p.vpt == 4) NB_V(4);
    NB_V(8);
  }
#undef NB_V
}

}  // namespace

// The launch of a planned product whose result is bfloat16 (gemm_stream_bf16.cu).  `plan` points
// to a StreamPlan of the caller's unit (the same struct: both units include this file).
int nb_gemm_stream_launch_bf16(const void* plan, const void* X, int x_is_f32, const float* gamma,
                               const float* beta, float eps, const void* W, const float* bias,
                               const float* residual, void* out, int M, int N, int K, int act,
                               cudaStream_t stream);
int nb_gemm_stream_bf16_set_wait_budget(long long cycles);
