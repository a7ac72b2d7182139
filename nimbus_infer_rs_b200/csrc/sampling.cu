// Token selection on the device: repetition penalty, greedy argmax, temperature sampling.
// One thread block per sequence; any vocabulary size.
//
// Reference (src/sampler.rs:163-217): logits are widened to f64; the penalty is applied
// first (:83-101); greedy takes the first index of the maximum (:172-180); otherwise the
// logits are divided by max(T, 1e-6), softmax is taken in f64 and the token is found by
// walking the cumulative sum until u * total is used up (:201-216).
#include "common.cuh"

namespace {

constexpr int THREADS = 256;

// For each distinct token of the sequence's history: logit > 0 ? logit / penalty
// : logit * penalty  (src/sampler.rs:83-101).  A token that occurs several times is
// penalised once: only its first occurrence acts.
__global__ void repetition_penalty_kernel(float* logits, int vocab,
                                          const int* history, int history_stride,
                                          const int* history_len, float penalty) {
  const int r = blockIdx.x;
  const int n = history_len[r];
  const int* hist = history + (size_t)r * history_stride;
  float* row = logits + (size_t)r * vocab;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int tok = hist[i];
    if (tok < 0 || tok >= vocab) continue;
    bool first = true;
    for (int j = 0; j < i; ++j)
      if (hist[j] == tok) { first = false; break; }
    if (!first) continue;
    const float v = row[tok];
    row[tok] = (v > 0.0f) ? (float)((double)v / (double)penalty) : (float)((double)v * (double)penalty);
  }
}

// A decode session keeps each sequence's generated tokens on the device: the token a live row
// runs in this step (the one selected in the step before) goes to the end of its history.
__global__ void history_append_kernel(int* history, int history_stride,
                                      int* history_len, const int* tokens,
                                      const int* row_slot, int n) {
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n || row_slot[i] < 0) return;
  const int len = history_len[i];
  if (len < history_stride) {
    history[(size_t)i * history_stride + len] = tokens[i];
    history_len[i] = len + 1;
  }
}

// First index of the maximum: an element replaces the best only if it is strictly greater
// (src/sampler.rs:173-179), so NaN never wins and ties go to the lower index.
__global__ void __launch_bounds__(THREADS)
argmax_kernel(const float* logits, int vocab, int* out) {
  __shared__ float s_val[THREADS];
  __shared__ int s_idx[THREADS];
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * vocab;
  // every thread starts from element 0, as the reference's scan does
  float best = row[0];
  int best_i = 0;
  for (int i = tid; i < vocab; i += THREADS) {
    const float v = row[i];
    if (v > best) { best = v; best_i = i; }
  }
  s_val[tid] = best;
  s_idx[tid] = best_i;
  __syncthreads();
  for (int off = THREADS / 2; off > 0; off >>= 1) {
    if (tid < off) {
      const float v = s_val[tid + off];
      const int i = s_idx[tid + off];
      if (v > s_val[tid] || (v == s_val[tid] && i < s_idx[tid])) {
        s_val[tid] = v;
        s_idx[tid] = i;
      }
    }
    __syncthreads();
  }
  if (tid == 0) out[r] = s_idx[0];
}

// The same over several CTAs per row (a large vocabulary scanned by one CTA is bound by
// latency).  Each CTA reduces its slice to one (value, index) pair, packs it into a 64-bit key
// whose unsigned order is "greater value first, then lower index", and merges it into the
// row's key with atomicMax; the CTA that arrives last for a row unpacks the winner and leaves
// key and counter at zero for the next launch.  NaN maps to the lowest key, so it never wins;
// if nothing beats it the answer is index 0, as in the single-CTA scan.
__device__ __forceinline__ unsigned long long argmax_key(float v, int idx) {
  if (v == 0.0f) v = 0.0f;                              // -0 and +0 tie, as they compare equal
  unsigned int b = __float_as_uint(v);
  b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);       // order-preserving map of finite floats
  if (v != v) b = 0u;                                    // NaN: lowest
  return ((unsigned long long)b << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)idx);
}

__global__ void __launch_bounds__(THREADS)
argmax_split_kernel(const float* logits, int vocab, int* out,
                    unsigned long long* keys, int* counters) {
  __shared__ unsigned long long s_key[THREADS / 32];
  __shared__ int s_last;
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int r = blockIdx.y, tid = threadIdx.x;
  const int per = (vocab + gridDim.x - 1) / gridDim.x;
  const int i0 = blockIdx.x * per, i1 = min(vocab, i0 + per);
  const float* row = logits + (size_t)r * vocab;
  unsigned long long best = 0ull;
  for (int i = i0 + tid; i < i1; i += THREADS) {
    const unsigned long long k = argmax_key(row[i], i);
    best = k > best ? k : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((tid & 31) == 0) s_key[tid >> 5] = best;
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < THREADS / 32; ++w) best = s_key[w] > best ? s_key[w] : best;
    atomicMax(&keys[r], best);
    __threadfence();
    const int old = atomicAdd(&counters[r], 1);
    s_last = (old == (int)gridDim.x - 1);
  }
  __syncthreads();
  if (s_last && tid == 0) {
    __threadfence();
    const unsigned long long k = atomicExch(&keys[r], 0ull);
    counters[r] = 0;
    // The sequential scan starts from element 0 and replaces it only by something strictly
    // greater: if element 0 is NaN nothing ever is, and the answer is 0.  Key 0 means every
    // element was NaN: index 0 as well.
    const float first = row[0];
    out[r] = ((k >> 32) == 0ull || first != first)
                 ? 0 : (int)(0xFFFFFFFFu - (unsigned)(k & 0xFFFFFFFFull));
  }
}

// Temperature sampling by inverse CDF in f64.  u[r] in [0,1) comes from the sequence's own
// generator on the host.  Each thread owns a contiguous segment of the vocabulary, so the
// walk over the cumulative sum visits the tokens in index order as the reference does.
__global__ void __launch_bounds__(THREADS)
sample_temperature_kernel(const float* logits, int vocab, float temperature,
                          const double* u, int* out) {
  __shared__ double s_red[THREADS];
  __shared__ int s_choice;
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * vocab;
  const double temp = fmax((double)temperature, 1e-6);
  const int per = (vocab + THREADS - 1) / THREADS;
  const int i0 = min(tid * per, vocab), i1 = min(i0 + per, vocab);

  double mx = -INFINITY;
  for (int i = i0; i < i1; ++i) mx = fmax(mx, (double)row[i] / temp);
  s_red[tid] = mx;
  __syncthreads();
  for (int off = THREADS / 2; off > 0; off >>= 1) {
    if (tid < off) s_red[tid] = fmax(s_red[tid], s_red[tid + off]);
    __syncthreads();
  }
  mx = s_red[0];
  __syncthreads();
  if (!isfinite(mx)) {  // all -inf (or NaN): the reference falls back to argmax -> index 0 scan
    if (tid == 0) {
      int best = 0;
      for (int i = 1; i < vocab; ++i)
        if ((double)row[i] / temp > (double)row[best] / temp) best = i;
      out[r] = best;
    }
    return;
  }
  double seg = 0.0;
  for (int i = i0; i < i1; ++i) seg += exp((double)row[i] / temp - mx);
  s_red[tid] = seg;
  if (tid == 0) s_choice = -1;
  __syncthreads();
  if (tid == 0) {
    double total = 0.0;
    for (int t = 0; t < THREADS; ++t) total += s_red[t];
    if (!isfinite(total) || total <= 0.0) {
      s_choice = -2;  // the reference returns token 0
    } else {
      double rem = u[r] * total;
      int t = 0;
      // skip whole segments that the remainder outlasts
      while (t < THREADS - 1 && rem - s_red[t] > 0.0) { rem -= s_red[t]; ++t; }
      s_choice = t;
      s_red[0] = rem;
    }
  }
  __syncthreads();
  if (s_choice == -2) { if (tid == 0) out[r] = 0; return; }
  if (tid == s_choice) {
    double rem = s_red[0];
    int pick = vocab - 1;
    for (int i = i0; i < vocab; ++i) {  // may run past the segment on rounding
      rem -= exp((double)row[i] / temp - mx);
      if (rem <= 0.0) { pick = i; break; }
    }
    out[r] = pick;
  }
}

// The n_keep largest logits of a row, with their indices: what top-k and top-p filtering can
// ever keep (src/sampler.rs:103-160 only ever keep the largest), so that the host's float64
// sampler works on a thousand candidates instead of the vocabulary.  One CTA per row finds the
// n_keep-th largest value by radix selection on order-preserving keys (three passes over the
// row, 11 + 11 + 10 bits), then writes out every element that is not smaller (in any order;
// ties at the threshold may make them more than n_keep: the count says how many, and what does
// not fit in `cap` is not written).  It also leaves the row's maximum and, in f64, the sum of
// exp((x - max) / temp) over the whole row: the softmax denominator the top-p rule needs.
// A NaN in the row gives count -1 (the caller then takes the full path).
constexpr int CAND_THREADS = 1024;

__device__ __forceinline__ unsigned int order_key(float v) {
  if (v == 0.0f) v = 0.0f;                              // -0 and +0 compare equal
  const unsigned int b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__global__ void __launch_bounds__(CAND_THREADS)
top_candidates_kernel(const float* logits, int vocab, int n_keep, int cap, double temp,
                      float* out_val, int* out_idx,
                      int* out_count, double* out_stats) {
  __shared__ unsigned int hist[2048];
  __shared__ unsigned int s_prefix, s_mask, s_remaining, s_count, s_nan;
  __shared__ float s_maxf[CAND_THREADS / 32];
  __shared__ double s_sum[CAND_THREADS / 32];
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * vocab;
  if (tid == 0) { s_prefix = 0u; s_mask = 0u; s_remaining = (unsigned)n_keep; s_count = 0u; s_nan = 0u; }
  __syncthreads();

  // maximum, NaN check
  float mx = -INFINITY;
  bool nan = false;
  for (int i = tid; i < vocab; i += CAND_THREADS) {
    const float v = row[i];
    nan |= (v != v);
    mx = fmaxf(mx, v);
  }
  mx = nb_warp_max(mx);
  if (nan) s_nan = 1u;
  if ((tid & 31) == 0) s_maxf[tid >> 5] = mx;
  __syncthreads();
  if (s_nan) {
    if (tid == 0) out_count[r] = -1;
    return;
  }
  mx = s_maxf[0];
  for (int w = 1; w < CAND_THREADS / 32; ++w) mx = fmaxf(mx, s_maxf[w]);
  // sum of exp((x - max) / temp) in f64
  double sum = 0.0;
  const double mxd = (double)mx / temp;
  for (int i = tid; i < vocab; i += CAND_THREADS) sum += exp((double)row[i] / temp - mxd);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if ((tid & 31) == 0) s_sum[tid >> 5] = sum;

  // radix selection of the n_keep-th largest key
  const int shifts[3] = {21, 10, 0};
  const int bits[3] = {11, 11, 10};
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = shifts[pass];
    const unsigned int nb = 1u << bits[pass];
    for (int i = tid; i < 2048; i += CAND_THREADS) hist[i] = 0u;
    __syncthreads();
    const unsigned int prefix = s_prefix, mask = s_mask;
    for (int i = tid; i < vocab; i += CAND_THREADS) {
      const unsigned int k = order_key(row[i]);
      if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & (nb - 1u)], 1u);
    }
    __syncthreads();
    if (tid == 0) {   // from the largest bin down: the bin that holds the element we look for
      unsigned int need = s_remaining, b = nb;
      while (b > 0u) {
        --b;
        if (hist[b] >= need) break;
        need -= hist[b];
      }
      s_remaining = need;
      s_prefix = prefix | (b << shift);
      s_mask = mask | ((nb - 1u) << shift);
    }
    __syncthreads();
  }
  const unsigned int threshold = s_prefix;
  for (int i = tid; i < vocab; i += CAND_THREADS) {
    const float v = row[i];
    if (order_key(v) >= threshold) {
      const unsigned int pos = atomicAdd(&s_count, 1u);
      if ((int)pos < cap) {
        out_val[(size_t)r * cap + pos] = v;
        out_idx[(size_t)r * cap + pos] = i;
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    double total = 0.0;
    for (int w = 0; w < CAND_THREADS / 32; ++w) total += s_sum[w];
    out_count[r] = (int)s_count;
    out_stats[2 * r] = (double)mx;
    out_stats[2 * r + 1] = total;
  }
}

// Top-k sampling wholly on the device (src/sampler.rs:103-116 then :181-215, top-p off): the
// k-th largest logit of the row is found by the same radix selection, everything below it is
// left out (ties at the threshold stay in, as in the reference), and the draw walks the
// cumulative sum of exp((x - max) / temp) over what is left in index order, in f64, with the
// u[r] that the sequence's own generator gave.  Each thread owns a contiguous piece of the
// vocabulary.  A row with a NaN gives -1 (the caller decides on the host).
__global__ void __launch_bounds__(CAND_THREADS)
sample_top_k_kernel(const float* logits, int vocab, int k, float temperature,
                    const double* u, int* out) {
  __shared__ unsigned int hist[2048];
  __shared__ unsigned int s_prefix, s_mask, s_remaining, s_nan;
  __shared__ float s_maxf[CAND_THREADS / 32];
  __shared__ double s_red[CAND_THREADS];
  __shared__ int s_choice;
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * vocab;
  if (tid == 0) { s_prefix = 0u; s_mask = 0u; s_remaining = (unsigned)k; s_nan = 0u; s_choice = -1; }
  __syncthreads();

  float mx = -INFINITY;
  bool nan = false;
  for (int i = tid; i < vocab; i += CAND_THREADS) {
    const float v = row[i];
    nan |= (v != v);
    mx = fmaxf(mx, v);
  }
  mx = nb_warp_max(mx);
  if (nan) s_nan = 1u;
  if ((tid & 31) == 0) s_maxf[tid >> 5] = mx;
  __syncthreads();
  if (s_nan) {
    if (tid == 0) out[r] = -1;
    return;
  }
  mx = s_maxf[0];
  for (int w = 1; w < CAND_THREADS / 32; ++w) mx = fmaxf(mx, s_maxf[w]);
  if (!isfinite(mx)) {   // all -inf, or a +inf: the reference takes the first maximum
    if (tid == 0) {
      int best = 0;
      for (int i = 1; i < vocab; ++i)
        if (row[i] > row[best]) best = i;
      out[r] = best;
    }
    return;
  }

  unsigned int threshold = 0u;   // keys at or above it are kept; 0 keeps everything
  if (k < vocab) {
    const int shifts[3] = {21, 10, 0};
    const int bits[3] = {11, 11, 10};
    for (int pass = 0; pass < 3; ++pass) {
      const int shift = shifts[pass];
      const unsigned int nb = 1u << bits[pass];
      for (int i = tid; i < 2048; i += CAND_THREADS) hist[i] = 0u;
      __syncthreads();
      const unsigned int prefix = s_prefix, mask = s_mask;
      for (int i = tid; i < vocab; i += CAND_THREADS) {
        const unsigned int key = order_key(row[i]);
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & (nb - 1u)], 1u);
      }
      __syncthreads();
      if (tid == 0) {   // from the largest bin down: the bin that holds the k-th largest
        unsigned int need = s_remaining, b = nb;
        while (b > 0u) {
          --b;
          if (hist[b] >= need) break;
          need -= hist[b];
        }
        s_remaining = need;
        s_prefix = prefix | (b << shift);
        s_mask = mask | ((nb - 1u) << shift);
      }
      __syncthreads();
    }
    threshold = s_prefix;
  }

  const double temp = fmax((double)temperature, 1e-6);
  const double mxd = (double)mx / temp;
  const int per = (vocab + CAND_THREADS - 1) / CAND_THREADS;
  const int i0 = min(tid * per, vocab), i1 = min(i0 + per, vocab);
  double seg = 0.0;
  for (int i = i0; i < i1; ++i)
    if (order_key(row[i]) >= threshold) seg += exp((double)row[i] / temp - mxd);
  s_red[tid] = seg;
  __syncthreads();
  if (tid == 0) {
    double total = 0.0;
    for (int t = 0; t < CAND_THREADS; ++t) total += s_red[t];
    if (!isfinite(total) || total <= 0.0) {
      s_choice = -2;   // the reference returns token 0
    } else {
      double rem = u[r] * total;
      int t = 0;
      while (t < CAND_THREADS - 1 && rem - s_red[t] > 0.0) { rem -= s_red[t]; ++t; }   // whole pieces
      s_choice = t;
      s_red[0] = rem;
    }
  }
  __syncthreads();
  if (s_choice == -2) {
    if (tid == 0) out[r] = 0;
    return;
  }
  if (tid == s_choice) {
    double rem = s_red[0];
    int pick = -1, last_kept = -1;
    for (int i = i0; i < vocab; ++i) {   // may run past the piece on rounding
      if (order_key(row[i]) < threshold) continue;
      last_kept = i;
      rem -= exp((double)row[i] / temp - mxd);
      if (rem <= 0.0) { pick = i; break; }
    }
    if (pick < 0) {   // rounding left a remainder after the last token: the last one kept
      pick = last_kept;
      for (int i = i0 - 1; pick < 0 && i >= 0; --i)
        if (order_key(row[i]) >= threshold) pick = i;
    }
    out[r] = pick;
  }
}

// Top-p sampling, with or without top-k (k <= TOPP_KEEP), on the device
// (src/sampler.rs:103-160, then :181-215).  The reference sorts the row in descending order
// (ties by index), walks the cumulative probability and drops a token when the mass before it
// minus its own exceeds p; both filters keep a prefix of that order.  Here the TOPP_KEEP largest
// logits are picked out by radix selection, sorted in shared memory (bitonic, value descending
// and index ascending in one 64-bit key), and one thread walks them as the reference does, in
// f64 and in the same order.  The last token kept defines the kept set for the whole row (a
// larger key, or the same value and no larger index), over which the draw then runs in index
// order as in the kernels above.  When the cut cannot be settled from the candidates (a flat
// distribution: more than TOPP_KEEP tokens survive) the row gets -2 and the caller decides on the
// host; a row with a NaN gets -1.
constexpr int TOPP_KEEP = 1024;
constexpr int TOPP_CAP = 2048;    // candidates the sort has room for (ties at the threshold)

__device__ __forceinline__ unsigned long long cand_key(float v, int i) {
  return ((unsigned long long)order_key(v) << 32) | (unsigned long long)(0xffffffffu - (unsigned)i);
}
__device__ __forceinline__ float key_value(unsigned long long c) {
  const unsigned int k = (unsigned int)(c >> 32);
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__global__ void __launch_bounds__(CAND_THREADS)
sample_top_p_kernel(const float* logits, int vocab, int k, float top_p, float temperature,
                    const double* u, int* out) {
  __shared__ double weight[TOPP_CAP];   // exp((x - max) / temp) of the sorted candidates ...
  unsigned int* hist = reinterpret_cast<unsigned int*>(weight);   // ... after the histograms
  __shared__ unsigned long long cand[TOPP_CAP];
  __shared__ unsigned int s_prefix, s_mask, s_remaining, s_nan, s_count;
  __shared__ float s_maxf[CAND_THREADS / 32];
  __shared__ double s_red[CAND_THREADS];
  __shared__ unsigned long long s_last_kept;
  __shared__ int s_choice;
  nb_grid_dependency_wait();
  nb_launch_dependents();
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * vocab;
  const int n_keep = min(TOPP_KEEP, vocab);
  if (tid == 0) {
    s_prefix = 0u; s_mask = 0u; s_remaining = (unsigned)n_keep; s_nan = 0u; s_count = 0u;
    s_choice = -1;
  }
  __syncthreads();

  float mx = -INFINITY;
  bool nan = false;
  for (int i = tid; i < vocab; i += CAND_THREADS) {
    const float v = row[i];
    nan |= (v != v);
    mx = fmaxf(mx, v);
  }
  mx = nb_warp_max(mx);
  if (nan) s_nan = 1u;
  if ((tid & 31) == 0) s_maxf[tid >> 5] = mx;
  __syncthreads();
  if (s_nan) {
    if (tid == 0) out[r] = -1;
    return;
  }
  mx = s_maxf[0];
  for (int w = 1; w < CAND_THREADS / 32; ++w) mx = fmaxf(mx, s_maxf[w]);
  if (!isfinite(mx)) {   // all -inf, or a +inf: the reference takes the first maximum
    if (tid == 0) {
      int best = 0;
      for (int i = 1; i < vocab; ++i)
        if (row[i] > row[best]) best = i;
      out[r] = best;
    }
    return;
  }
  const double temp = fmax((double)temperature, 1e-6);
  const double mxd = (double)mx / temp;

  // the softmax denominator over the whole row (used when top-k is off)
  double sum = 0.0;
  for (int i = tid; i < vocab; i += CAND_THREADS) sum += exp((double)row[i] / temp - mxd);
  s_red[tid] = sum;

  // the n_keep-th largest key, then every element that is not smaller into `cand`
  {
    const int shifts[3] = {21, 10, 0};
    const int bits[3] = {11, 11, 10};
    for (int pass = 0; pass < 3; ++pass) {
      const int shift = shifts[pass];
      const unsigned int nb = 1u << bits[pass];
      for (int i = tid; i < 2048; i += CAND_THREADS) hist[i] = 0u;
      __syncthreads();
      const unsigned int prefix = s_prefix, mask = s_mask;
      for (int i = tid; i < vocab; i += CAND_THREADS) {
        const unsigned int key = order_key(row[i]);
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & (nb - 1u)], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        unsigned int need = s_remaining, b = nb;
        while (b > 0u) {
          --b;
          if (hist[b] >= need) break;
          need -= hist[b];
        }
        s_remaining = need;
        s_prefix = prefix | (b << shift);
        s_mask = mask | ((nb - 1u) << shift);
      }
      __syncthreads();
    }
  }
  const unsigned int threshold = s_prefix;
  for (int i = tid; i < TOPP_CAP; i += CAND_THREADS) cand[i] = 0ull;
  __syncthreads();
  for (int i = tid; i < vocab; i += CAND_THREADS) {
    const float v = row[i];
    if (order_key(v) >= threshold) {
      const unsigned int pos = atomicAdd(&s_count, 1u);
      if (pos < (unsigned)TOPP_CAP) cand[pos] = cand_key(v, i);
    }
  }
  __syncthreads();
  const int n = (int)s_count;
  if (n > TOPP_CAP) {   // more ties at the threshold than the sort has room for
    if (tid == 0) out[r] = -2;
    return;
  }
  // bitonic sort, descending (empty places are zero: they end up last)
  for (int size = 2; size <= TOPP_CAP; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = tid; t < TOPP_CAP / 2; t += CAND_THREADS) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool down = (lo & size) == 0;   // this run is sorted descending
        const unsigned long long a = cand[lo], b = cand[hi];
        if ((a < b) == down) {
          cand[lo] = b;
          cand[hi] = a;
        }
      }
      __syncthreads();
    }
  }

  // the candidates' weights, by everybody: the walk below is then additions only
  for (int j = tid; j < n; j += CAND_THREADS) weight[j] = exp((double)key_value(cand[j]) / temp - mxd);
  __syncthreads();
  if (tid == 0) {
    double row_sum = 0.0;
    for (int t = 0; t < CAND_THREADS; ++t) row_sum += s_red[t];
    // the universe the probabilities are taken over: the row, or what top-k leaves of it
    int m = n;
    bool complete = (n == vocab);   // every token of the universe is among the candidates
    double S = row_sum;
    if (k > 0 && k < vocab) {
      const int kk = min(k, n);
      const unsigned int kth = (unsigned int)(cand[kk - 1] >> 32);
      m = kk;
      while (m < n && (unsigned int)(cand[m] >> 32) == kth) ++m;   // ties at the k-th stay
      complete = true;   // all of them are at or above the candidates' threshold: none is missing
      S = 0.0;
      for (int j = 0; j < m; ++j) S += weight[j];
    }
    int kept = -1;
    if (!(S > 0.0) || !isfinite(S)) {
      kept = -3;   // the reference's draw returns token 0 when the total is not a positive number
    } else if (top_p <= 0.0f) {
      kept = 1;    // the first maximum alone
    } else {
      const double p = (double)top_p;
      double cum = 0.0, prob = 0.0;
      for (int j = 0; j < m; ++j) {
        prob = weight[j] / S;
        if (cum - prob > p) { kept = j; break; }
        cum += prob;
      }
      if (kept < 0) {
        // nobody among the candidates is dropped.  A token outside them weighs no more than the
        // last candidate: it is dropped for sure if even that weight would be.
        if (complete || cum - prob > p) kept = m;
        else kept = -2;
      }
    }
    if (kept == -2) {
      out[r] = -2;
      s_choice = -3;
    } else if (kept == -3) {
      out[r] = 0;
      s_choice = -3;
    } else {
      s_last_kept = cand[kept - 1];
    }
  }
  __syncthreads();
  if (s_choice == -3) return;
  const unsigned long long last_kept = s_last_kept;

  const int per = (vocab + CAND_THREADS - 1) / CAND_THREADS;
  const int i0 = min(tid * per, vocab), i1 = min(i0 + per, vocab);
  double seg = 0.0;
  for (int i = i0; i < i1; ++i)
    if (cand_key(row[i], i) >= last_kept) seg += exp((double)row[i] / temp - mxd);
  __syncthreads();
  s_red[tid] = seg;
  __syncthreads();
  if (tid == 0) {
    double total = 0.0;
    for (int t = 0; t < CAND_THREADS; ++t) total += s_red[t];
    if (!isfinite(total) || total <= 0.0) {
      s_choice = -2;
    } else {
      double rem = u[r] * total;
      int t = 0;
      while (t < CAND_THREADS - 1 && rem - s_red[t] > 0.0) { rem -= s_red[t]; ++t; }
      s_choice = t;
      s_red[0] = rem;
    }
  }
  __syncthreads();
  if (s_choice == -2) {
    if (tid == 0) out[r] = 0;
    return;
  }
  if (tid == s_choice) {
    double rem = s_red[0];
    int pick = -1, last = -1;
    for (int i = i0; i < vocab; ++i) {
      if (cand_key(row[i], i) < last_kept) continue;
      last = i;
      rem -= exp((double)row[i] / temp - mxd);
      if (rem <= 0.0) { pick = i; break; }
    }
    if (pick < 0) {
      pick = last;
      for (int i = i0 - 1; pick < 0 && i >= 0; --i)
        if (cand_key(row[i], i) >= last_kept) pick = i;
    }
    out[r] = pick;
  }
}

}  // namespace

// n_keep <= cap.  out_val / out_idx: [n_rows, cap]; out_count: [n_rows]; out_stats: [n_rows, 2]
// (maximum, sum of exp((x - max) / temp)).  Fewer than n_keep elements in a row: all of them.
NB_EXPORT int nb_top_candidates(const float* logits, int n_rows, int vocab, int n_keep, int cap,
                                double temp, float* out_val, int* out_idx, int* out_count,
                                double* out_stats, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(vocab > 0 && n_keep >= 1 && cap >= n_keep && temp > 0.0, NB_ERR_BAD_ARG,
             "top_candidates: bad sizes vocab=%d keep=%d cap=%d", vocab, n_keep, cap);
  top_candidates_kernel<<<n_rows, CAND_THREADS, 0, stream>>>(logits, vocab, n_keep, cap, temp, out_val,
                                                             out_idx, out_count, out_stats);
  NB_CHECK_LAUNCH("top_candidates");
  return 0;
}

// 1 <= k; k >= vocab keeps the whole row.  u: one f64 in [0, 1) per row; out: the token, or -1
// for a row with a NaN.
NB_EXPORT int nb_sample_top_k(const float* logits, int n_rows, int vocab, int k, float temperature,
                              const double* u, int* out, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(vocab > 0 && k >= 1, NB_ERR_BAD_ARG, "sample_top_k: bad sizes vocab=%d k=%d", vocab, k);
  NB_CUDA(nb_launch(sample_top_k_kernel, dim3(n_rows), dim3(CAND_THREADS), 0, stream, logits, vocab, k,
                    temperature, u, out));
  NB_CHECK_LAUNCH("sample_top_k");
  return 0;
}

// The most top-k that nb_sample_top_p takes together with top-p (0 = top-k off).
NB_EXPORT int nb_sample_top_p_max_k() { return TOPP_KEEP; }

// k = 0: top-p alone; else 1 <= k <= nb_sample_top_p_max_k().  out: the token; -1 for a row with
// a NaN, -2 for a row whose cut lies beyond the candidates (the caller decides on the host).
NB_EXPORT int nb_sample_top_p(const float* logits, int n_rows, int vocab, int k, float top_p,
                              float temperature, const double* u, int* out, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(vocab > 0 && k >= 0 && k <= TOPP_KEEP, NB_ERR_BAD_ARG,
             "sample_top_p: bad sizes vocab=%d k=%d (at most %d)", vocab, k, TOPP_KEEP);
  NB_CUDA(nb_launch(sample_top_p_kernel, dim3(n_rows), dim3(CAND_THREADS), 0, stream, logits, vocab, k,
                    top_p, temperature, u, out));
  NB_CHECK_LAUNCH("sample_top_p");
  return 0;
}

// history: [n_rows, history_stride]; a row whose history is full is left as it is.
NB_EXPORT int nb_history_append(int* history, int history_stride, int* history_len, const int* tokens,
                                const int* row_slot, int n_rows, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(history_stride >= 1, NB_ERR_BAD_ARG, "history_append: no room (stride %d)", history_stride);
  NB_CUDA(nb_launch(history_append_kernel, dim3((n_rows + 127) / 128), dim3(128), 0, stream, history,
                    history_stride, history_len, tokens, row_slot, n_rows));
  NB_CHECK_LAUNCH("history_append");
  return 0;
}

NB_EXPORT int nb_repetition_penalty(float* logits, int n_rows, int vocab, const int* history,
                                    int history_stride, const int* history_len, float penalty,
                                    cudaStream_t stream) {
  if (n_rows == 0 || penalty == 1.0f) return 0;
  repetition_penalty_kernel<<<n_rows, 128, 0, stream>>>(logits, vocab, history, history_stride,
                                                        history_len, penalty);
  NB_CHECK_LAUNCH("repetition_penalty");
  return 0;
}

// Scratch: `keys` (8 bytes per row) and `counters` (4 bytes per row), zero before the first
// use; every launch leaves them at zero.  n_ctas CTAs scan each row.
NB_EXPORT int nb_argmax_split(const float* logits, int n_rows, int vocab, int* out,
                              unsigned long long* keys, int* counters, int n_ctas,
                              cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(vocab > 0 && n_ctas >= 1 && n_rows <= 65535, NB_ERR_BAD_ARG,
             "argmax_split: bad sizes rows=%d vocab=%d ctas=%d", n_rows, vocab, n_ctas);
  NB_REQUIRE(keys && counters, NB_ERR_BAD_ARG, "argmax_split: scratch missing");
  NB_CUDA(nb_launch(argmax_split_kernel, dim3(n_ctas, n_rows), dim3(THREADS), 0, stream, logits,
                    vocab, out, keys, counters));
  NB_CHECK_LAUNCH("argmax_split");
  return 0;
}

NB_EXPORT int nb_argmax(const float* logits, int n_rows, int vocab, int* out, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(vocab > 0, NB_ERR_BAD_ARG, "argmax: empty vocabulary");
  NB_CUDA(nb_launch(argmax_kernel, dim3(n_rows), dim3(THREADS), 0, stream, logits, vocab, out));
  NB_CHECK_LAUNCH("argmax");
  return 0;
}

NB_EXPORT int nb_sample_temperature(const float* logits, int n_rows, int vocab, float temperature,
                                    const double* u, int* out, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NB_REQUIRE(vocab > 0, NB_ERR_BAD_ARG, "sample_temperature: empty vocabulary");
  NB_CUDA(nb_launch(sample_temperature_kernel, dim3(n_rows), dim3(THREADS), 0, stream, logits, vocab,
                    temperature, u, out));
  NB_CHECK_LAUNCH("sample_temperature");
  return 0;
}
