// Sampling on the device, one block per row of logits.
//
// Greedy: the first maximum wins (src/l5_model.c:610-614 of AnonymoDGH/gguf2bin).
// Temperature: logits /= temp; softmax; the first i with r <= cumulative sum, else the
// last id (src/l5_model.c:615-619).  The reference draws r from rand(), seeded by the
// clock; here r comes from a Philox4x32-10 stream per sequence, keyed by the per-slot
// record {seed_lo, seed_hi, stream, draws}: counter = (draws, stream, 0, 0), and
// r = (first output word >> 8) / 2^24.  The draw count advances by one per sampled
// token, so a sequence's choices do not depend on the batch it is in.
//
// Filtered sampling (src/main.c:197-268): repeat penalty on the distinct recent ids
// (v > 0 ? v / R : v * R), then logits / temp in descending order (ties: lower id
// first), the best top_k kept, softmax over the kept, the shortest prefix whose
// cumulative sum reaches top_p kept and renormalised, then the first kept entry with
// r <= cumulative sum.  With a top_k of up to 2,048 the kept entries are listed and sorted
// (two counting passes over the order-preserving integer image of the logits find where the
// k-th largest lies); without a top_k, weighted radix descents over that image do the same
// without a sort of the vocabulary.
#include "common.cuh"

G2B_DEFINE_LAST_ERROR

#define SAMPLE_THREADS 1024

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t out[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// Draws the next uniform number of a slot's stream and advances the stream.
__device__ __forceinline__ float next_uniform(int *seq_state, int slot, int words) {
  int *rec = seq_state + (size_t)slot * words;
  uint32_t o[4];
  philox4x32_10((uint32_t)rec[3], (uint32_t)rec[2], 0u, 0u, (uint32_t)rec[0], (uint32_t)rec[1], o);
  rec[3] += 1;
  return (float)(o[0] >> 8) * (1.0f / 16777216.0f);
}

// ---- block argmax: lowest index among equal maxima ---------------------------
__device__ int block_argmax(const float *row, int V, float inv_temp, float *best_out) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i] * inv_temp;
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { s_val[warp] = bv; s_idx[warp] = bi; }
  __syncthreads();
  const int n_warps = (blockDim.x + 31) >> 5;
  bv = lane < n_warps ? s_val[lane] : -INFINITY;
  bi = lane < n_warps ? s_idx[lane] : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if (best_out) *best_out = bv;
  return bi == 0x7fffffff ? 0 : bi;   // all-NaN row: id 0, as a scan from index 0 gives
}

// ---- greedy / plain temperature ---------------------------------------------
// Temperature: warp w owns the contiguous range [w C, (w + 1) C) of the row, C a multiple of
// 32, and reads it 32 consecutive entries at a time (whole cache lines: a thread per contiguous
// chunk read 30 times the bytes).  The cumulative sum runs in index order: over the warps'
// totals to the warp whose range holds the crossing, over that warp's steps of 32 to the step,
// and by a prefix sum over its lanes to the entry.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float *__restrict__ logits, int V, int ld, float temp, int *seq_state,
                   int state_words, const int *__restrict__ slots, int *__restrict__ out_ids) {
  pdl_launch();
  pdl_wait();
  __shared__ float s_wtot[SAMPLE_THREADS / 32];
  __shared__ float s_r, s_total, s_before;
  __shared__ int s_warp, s_choice;
  const float *row = logits + (size_t)blockIdx.x * ld;
  if (temp <= 0.f) {
    const int id = block_argmax(row, V, 1.f, nullptr);
    if (threadIdx.x == 0) out_ids[blockIdx.x] = id;
    return;
  }
  float mx;
  block_argmax(row, V, 1.f, &mx);                  // max of the raw logits
  mx = mx / temp;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_warps = blockDim.x >> 5;
  const int C = ((V + n_warps - 1) / n_warps + 31) / 32 * 32;
  const int begin = min(V, warp * C), end = min(V, begin + C);
  float part = 0.f;
  for (int i = begin + lane; i < end; i += 32) part += expf(row[i] / temp - mx);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if (lane == 0) s_wtot[warp] = part;
  __syncthreads();
  if (threadIdx.x == 0) {
    const float r = next_uniform(seq_state, slots[blockIdx.x], state_words);
    float total = 0.f;
    for (int w = 0; w < n_warps; ++w) total += s_wtot[w];
    // first i with r <= c_i where c_i = (e_0 + ... + e_i) / total
    float c = 0.f;
    int owner = -1;
    for (int w = 0; w < n_warps; ++w) {
      if (s_wtot[w] > 0.f && r <= (c + s_wtot[w]) / total) { owner = w; break; }
      c += s_wtot[w];
    }
    s_r = r; s_total = total; s_before = c; s_warp = owner;
    s_choice = V - 1;
  }
  __syncthreads();
  if (warp == s_warp) {
    const float r = s_r, total = s_total;
    float c = s_before;
    int choice = end - 1;                          // rounding: stay inside the owner's range
    for (int i0 = begin; i0 < end; i0 += 32) {
      const int i = i0 + lane;
      const float e = i < end ? expf(row[i] / temp - mx) : 0.f;
      float incl = e;                              // inclusive prefix sum over the lanes
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      const bool hit = i < end && r <= (c + incl) / total;
      const unsigned ballot = __ballot_sync(0xffffffffu, hit);
      if (ballot) {
        choice = i0 + __ffs(ballot) - 1;
        break;
      }
      c += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) s_choice = choice;
  }
  __syncthreads();
  if (threadIdx.x == 0) out_ids[blockIdx.x] = s_choice;
}

extern "C" int g2b_sample_rows(const float *logits, int R, int V, int ld, float temp,
                               int *seq_state, int state_words, const int *slots, int *out_ids,
                               cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || ld < V) G2B_REFUSE("sample_rows: bad sizes V=%d ld=%d", V, ld);
  if (temp > 0.f && (!seq_state || !slots || state_words < 4))
    G2B_REFUSE("sample_rows: temperature sampling needs the per-slot state");
  g2b_launch(sample_rows_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream, logits, V, ld, temp, seq_state,
                                                       state_words, slots, out_ids);
  return g2b_check_launch("sample_rows");
}

// ---- greedy over many blocks per row ---------------------------------------------
// A vocabulary of 150k entries and a handful of rows leave most of the GPU idle when a
// row is one block's work.  Stage 1: grid (row, split), each block reduces a contiguous
// slice of the row to (value, index); stage 2: one block per row picks among the slices.
// The first maximum wins at both stages, as a scan from index 0 would find it.
#define ARGMAX_SPLITS 64

__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float *__restrict__ logits, int V, int ld, float *__restrict__ part_val,
                      int *__restrict__ part_idx) {
  pdl_launch();
  pdl_wait();
  const float *row = logits + (size_t)blockIdx.x * ld;
  const int per = (V + ARGMAX_SPLITS - 1) / ARGMAX_SPLITS;
  const int begin = min(V, (int)blockIdx.y * per), end = min(V, begin + per);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const float v = row[i];
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
  __shared__ float s_val[8];
  __shared__ int s_idx[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { s_val[warp] = bv; s_idx[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (s_val[w] > bv || (s_val[w] == bv && s_idx[w] < bi)) { bv = s_val[w]; bi = s_idx[w]; }
    part_val[blockIdx.x * ARGMAX_SPLITS + blockIdx.y] = bv;
    part_idx[blockIdx.x * ARGMAX_SPLITS + blockIdx.y] = bi;
  }
}

__global__ void __launch_bounds__(ARGMAX_SPLITS)
argmax_final_kernel(const float *__restrict__ part_val, const int *__restrict__ part_idx,
                    int *__restrict__ out_ids) {
  pdl_launch();
  pdl_wait();
  float bv = part_val[blockIdx.x * ARGMAX_SPLITS + threadIdx.x];
  int bi = part_idx[blockIdx.x * ARGMAX_SPLITS + threadIdx.x];
  __shared__ float s_val[ARGMAX_SPLITS / 32];
  __shared__ int s_idx[ARGMAX_SPLITS / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = bv; s_idx[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < ARGMAX_SPLITS / 32; ++w)
      if (s_val[w] > bv || (s_val[w] == bv && s_idx[w] < bi)) { bv = s_val[w]; bi = s_idx[w]; }
    out_ids[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
}

// scratch: part_val float [R * 64], part_idx int [R * 64]
extern "C" int g2b_argmax_rows(const float *logits, int R, int V, int ld, float *part_val,
                               int *part_idx, int *out_ids, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || ld < V) G2B_REFUSE("argmax_rows: bad sizes V=%d ld=%d", V, ld);
  if (R > 65535) G2B_REFUSE("argmax_rows: %d rows", R);
  g2b_launch(argmax_partial_kernel, dim3(R, ARGMAX_SPLITS), dim3(256), 0, stream, logits, V, ld,
             part_val, part_idx);
  g2b_launch(argmax_final_kernel, dim3(R), dim3(ARGMAX_SPLITS), 0, stream, part_val, part_idx, out_ids);
  return g2b_check_launch("argmax_rows");
}

// ---- filtered sampling: repeat penalty, top-k, top-p ---------------------------
// Order-preserving map float -> uint32 (larger float, larger key).
__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One weighted radix descent.  Among the entries that pass `admit` (key below the
// admitted bound, or equal to it with few enough equal-key predecessors: see the
// caller), walk keys from the largest down and find the key at which the running weight
// first reaches `target`.  Returns that key and the weight of all entries with a larger
// key through shared memory.  weight(i) is 1 for counting or e_i for mass.
struct Descent {
  uint32_t key;        // key where the running weight reaches the target
  float above;         // weight of admitted entries with key > key
};

template <bool MASS>
__device__ Descent radix_descent(const float *row, int V, float inv_temp, float mx,
                                 uint32_t bound_key, bool bounded, float target, float *hist) {
  // hist: 256 floats in shared memory
  __shared__ uint32_t s_prefix;
  __shared__ float s_above;
  if (threadIdx.x == 0) { s_prefix = 0u; s_above = 0.f; }
  __syncthreads();
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0.f;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = row[i] * inv_temp;
      const uint32_t k = order_key(v);
      if (bounded && k < bound_key) continue;      // below the kept set
      if ((k & mask) != (prefix & mask)) continue;
      const float w = MASS ? expf(v - mx) : 1.f;
      atomicAdd(&hist[(k >> shift) & 0xffu], w);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float run = s_above;
      int chosen = -1, last = 0;
      for (int d = 255; d >= 0; --d) {
        if (!(hist[d] > 0.f)) continue;            // empty buckets are never chosen
        last = d;
        if (run + hist[d] >= target) { chosen = d; break; }
        run += hist[d];
      }
      if (chosen < 0) {                            // rounding left the target just above the total
        chosen = last;
        run -= hist[last];
      }
      s_above = run;
      s_prefix = prefix | ((uint32_t)chosen << shift);
    }
    __syncthreads();
  }
  Descent out;
  out.key = s_prefix;
  out.above = s_above;
  __syncthreads();
  return out;
}

// Among entries whose key equals `key`, in index order, the index at which
// `above + running weight` first reaches target.  All threads look for the equal-key entries
// (ties are rare: usually there is one) and list their indices; thread 0 puts the list in
// index order and walks it.  Only when the list overflows (thousands of equal logits) does
// thread 0 walk the whole row.
constexpr int TIE_CAP = 1024;
template <bool MASS>
__device__ int tie_walk(const float *row, int V, float inv_temp, float mx, uint32_t key,
                        float above, float target, int *tie_list) {
  __shared__ int s_idx, s_n;
  if (threadIdx.x == 0) s_n = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    if (order_key(row[i] * inv_temp) == key) {
      const int j = atomicAdd(&s_n, 1);
      if (j < TIE_CAP) tie_list[j] = i;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = above;
    int idx = -1;
    const int n = s_n;
    if (n <= TIE_CAP) {
      for (int a = 1; a < n; ++a) {                 // insertion sort: index order
        const int v = tie_list[a];
        int b = a - 1;
        while (b >= 0 && tie_list[b] > v) { tie_list[b + 1] = tie_list[b]; --b; }
        tie_list[b + 1] = v;
      }
      for (int a = 0; a < n; ++a) {
        const int i = tie_list[a];
        run += MASS ? expf(row[i] * inv_temp - mx) : 1.f;
        idx = i;
        if (run >= target) break;
      }
    } else {
      for (int i = 0; i < V; ++i) {
        const float v = row[i] * inv_temp;
        if (order_key(v) != key) continue;
        run += MASS ? expf(v - mx) : 1.f;
        idx = i;
        if (run >= target) break;
      }
    }
    s_idx = idx;
  }
  __syncthreads();
  const int idx = s_idx;
  __syncthreads();
  return idx;
}

// Weight of admitted entries: key > bound_key, or key == bound_key and index <= tie_idx.
__device__ float admitted_mass(const float *row, int V, float inv_temp, float mx,
                               uint32_t bound_key, int tie_idx, bool bounded, float *scratch) {
  float part = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i] * inv_temp;
    const uint32_t k = order_key(v);
    if (bounded && (k < bound_key || (k == bound_key && i > tie_idx))) continue;
    part += expf(v - mx);
  }
  return block_sum(part, scratch);
}

// ---- top-k as a short list --------------------------------------------------------------
// With a top_k of a few dozen the kept set is tiny: two counting passes over the row (11 bits
// of the key each) find the 22-bit prefix of the k-th largest key, a third lists every entry
// at or above that prefix (the k - 1 larger ones and those that share it: usually a handful),
// the list is sorted (key descending, then index ascending: the reference's order), cut to k,
// and top-p and the draw are walks over at most k entries.  When the list would overflow
// (thousands of logits sharing 22 bits) the caller takes the descents over the whole row.
constexpr int LIST_CAP = 2048;
struct ShortList {
  uint32_t key[LIST_CAP];
  int idx[LIST_CAP];
  float e[LIST_CAP];
  int hist[2048];
};

// Returns the number of listed entries (sorted, at least top_k of them), or -1 on overflow.
__device__ int list_top_k(const float *row, int V, float inv_temp, int top_k, ShortList &L) {
  __shared__ uint32_t s_prefix;
  __shared__ int s_above, s_n;
  if (threadIdx.x == 0) { s_prefix = 0u; s_above = 0; s_n = 0; }
  __syncthreads();
  for (int pass = 0; pass < 2; ++pass) {
    const int shift = pass == 0 ? 21 : 10;
    for (int i = threadIdx.x; i < 2048; i += blockDim.x) L.hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const uint32_t k = order_key(row[i] * inv_temp);
      if (pass == 1 && (k >> 21) != (prefix >> 21)) continue;
      // most logits share a few bins: the lanes of a warp that hit the same bin add once
      const int bin = (int)((k >> shift) & 0x7ffu);
      const unsigned peers = __match_any_sync(__activemask(), bin);
      if ((int)(threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&L.hist[bin], __popc(peers));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int run = s_above, chosen = 0;
      for (int d = 2047; d >= 0; --d) {
        if (run + L.hist[d] >= top_k) { chosen = d; break; }
        run += L.hist[d];
      }
      s_above = run;
      s_prefix = prefix | ((uint32_t)chosen << shift);
      if (pass == 1) s_n = run + L.hist[chosen];        // entries at or above the 22-bit prefix
    }
    __syncthreads();
  }
  const int total = s_n;
  if (total > LIST_CAP || total < top_k) return -1;
  const uint32_t floor22 = s_prefix >> 10;
  __syncthreads();
  if (threadIdx.x == 0) s_n = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const uint32_t k = order_key(row[i] * inv_temp);
    if ((k >> 10) >= floor22) {
      const int j = atomicAdd(&s_n, 1);
      if (j < LIST_CAP) { L.key[j] = k; L.idx[j] = i; }
    }
  }
  __syncthreads();
  const int n = s_n;
  if (n > LIST_CAP) return -1;
  int n2 = 1;
  while (n2 < n) n2 <<= 1;
  for (int i = n + threadIdx.x; i < n2; i += blockDim.x) { L.key[i] = 0u; L.idx[i] = 0x7fffffff; }
  __syncthreads();
  // bitonic sort: key descending, index ascending
  for (int k = 2; k <= n2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < n2; i += blockDim.x) {
        const int p = i ^ j;
        if (p > i) {
          const bool up = (i & k) == 0;             // this pair in "descending" order
          const uint32_t ka = L.key[i], kb = L.key[p];
          const int ia = L.idx[i], ib = L.idx[p];
          const bool a_first = ka > kb || (ka == kb && ia < ib);     // a belongs before b
          if (a_first != up) {
            L.key[i] = kb; L.key[p] = ka;
            L.idx[i] = ib; L.idx[p] = ia;
          }
        }
      }
      __syncthreads();
    }
  }
  return n;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_filtered_kernel(float *__restrict__ logits, int V, int ld, float temp, int top_k,
                       float top_p, float penalty, const int *__restrict__ recent, int recent_ld,
                       const int *__restrict__ recent_n, int *seq_state, int state_words,
                       const int *__restrict__ slots, int *__restrict__ out_ids) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  __shared__ float s_r;
  __shared__ ShortList L;
  float *hist = L.e;                                // the descents' 256 bins and the tie list live in the list's arrays
  int *tie_list = L.idx;
  float *row = logits + (size_t)blockIdx.x * ld;

  // repeat penalty, each distinct id once (src/main.c:204-223)
  if (penalty != 1.f && recent) {
    const int *rc = recent + (size_t)blockIdx.x * recent_ld;
    const int n = min(max(recent_n[blockIdx.x], 0), recent_ld);   // never past the row
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int id = rc[i];
      if (id < 0 || id >= V) continue;
      bool first = true;
      for (int j = 0; j < i; ++j) if (rc[j] == id) { first = false; break; }
      if (!first) continue;
      const float v = row[id];
      row[id] = v > 0.f ? v / penalty : v * penalty;
    }
    __syncthreads();
  }
  if (temp <= 0.f) {
    const int id = block_argmax(row, V, 1.f, nullptr);
    if (threadIdx.x == 0) out_ids[blockIdx.x] = id;
    return;
  }
  const float inv_temp = 1.f / temp;
  float mx;
  block_argmax(row, V, inv_temp, &mx);

  if (top_k > 0 && top_k < V && top_k <= LIST_CAP) {
    const int n = list_top_k(row, V, inv_temp, top_k, L);
    if (n >= 0) {
      const int n_keep0 = min(n, top_k);
      for (int j = threadIdx.x; j < n_keep0; j += blockDim.x) L.e[j] = expf(row[L.idx[j]] * inv_temp - mx);
      __syncthreads();
      if (threadIdx.x == 0) {
        int n_keep = n_keep0;
        float kept = 0.f;
        for (int j = 0; j < n_keep; ++j) kept += L.e[j];
        if (top_p < 1.f) {
          // shortest prefix (descending) whose cumulative probability reaches top_p
          const float target = top_p * kept;
          float run = 0.f;
          for (int j = 0; j < n_keep; ++j) {
            run += L.e[j];
            if (run >= target) { n_keep = j + 1; break; }
          }
          kept = 0.f;
          for (int j = 0; j < n_keep; ++j) kept += L.e[j];
        }
        const float target = next_uniform(seq_state, slots[blockIdx.x], state_words) * kept;
        float run = 0.f;
        int pick = L.idx[n_keep - 1];
        for (int j = 0; j < n_keep; ++j) {
          run += L.e[j];
          if (run >= target) { pick = L.idx[j]; break; }
        }
        out_ids[blockIdx.x] = pick;
      }
      return;
    }
    __syncthreads();
  }

  // kept set: key > bound_key, or key == bound_key with index <= tie_idx
  bool bounded = false;
  uint32_t bound_key = 0u;
  int tie_idx = V;
  if (top_k > 0 && top_k < V) {
    const Descent d = radix_descent<false>(row, V, inv_temp, mx, 0u, false, (float)top_k, hist);
    tie_idx = tie_walk<false>(row, V, inv_temp, mx, d.key, d.above, (float)top_k, tie_list);
    bound_key = d.key;
    bounded = true;
  }
  float kept = admitted_mass(row, V, inv_temp, mx, bound_key, tie_idx, bounded, scratch);
  if (top_p < 1.f) {
    // shortest prefix (descending) whose cumulative probability reaches top_p
    const float target = top_p * kept;
    const Descent d = radix_descent<true>(row, V, inv_temp, mx, bound_key, bounded, target, hist);
    int t2 = tie_walk<true>(row, V, inv_temp, mx, d.key, d.above, target, tie_list);
    if (bounded && d.key == bound_key && t2 > tie_idx) t2 = tie_idx;
    bound_key = d.key;
    tie_idx = t2;
    bounded = true;
    kept = admitted_mass(row, V, inv_temp, mx, bound_key, tie_idx, bounded, scratch);
  }
  if (threadIdx.x == 0) s_r = next_uniform(seq_state, slots[blockIdx.x], state_words);
  __syncthreads();
  const float target = s_r * kept;
  const Descent d = radix_descent<true>(row, V, inv_temp, mx, bound_key, bounded, target, hist);
  int choice = tie_walk<true>(row, V, inv_temp, mx, d.key, d.above, target, tie_list);
  if (bounded && d.key == bound_key && choice > tie_idx) choice = tie_idx;
  if (threadIdx.x == 0) out_ids[blockIdx.x] = choice < 0 ? 0 : choice;
}

// recent: [R, recent_ld] ids, recent_n[R] how many are valid; logits are modified in
// place by the penalty.
extern "C" int g2b_sample_filtered(float *logits, int R, int V, int ld, float temp, int top_k,
                                   float top_p, float penalty, const int *recent, int recent_ld,
                                   const int *recent_n, int *seq_state, int state_words,
                                   const int *slots, int *out_ids, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || ld < V) G2B_REFUSE("sample_filtered: bad sizes V=%d ld=%d", V, ld);
  if (!(top_p > 0.f)) G2B_REFUSE("sample_filtered: top_p must be in (0, 1], got %g", top_p);
  if (!(penalty > 0.f)) G2B_REFUSE("sample_filtered: repeat penalty must be positive, got %g", penalty);
  if (temp > 0.f && (!seq_state || !slots || state_words < 4))
    G2B_REFUSE("sample_filtered: temperature sampling needs the per-slot state");
  g2b_launch(sample_filtered_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream, 
      logits, V, ld, temp, top_k, top_p, penalty, recent, recent_ld, recent_n, seq_state,
      state_words, slots, out_ids);
  return g2b_check_launch("sample_filtered");
}

// Seeds the per-slot records of the given slots: {seed_lo, seed_hi, stream, draws = 0}.
__global__ void seed_slots_kernel(int *seq_state, int words, const int *slots, const int *streams,
                                  int n, uint32_t seed_lo, uint32_t seed_hi) {
  pdl_launch();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int *rec = seq_state + (size_t)slots[i] * words;
  rec[0] = (int)seed_lo; rec[1] = (int)seed_hi; rec[2] = streams[i]; rec[3] = 0;
}

extern "C" int g2b_seed_slots(int *seq_state, int words, const int *slots, const int *streams,
                              int n, unsigned long long seed, cudaStream_t stream) {
  if (n <= 0) return 0;
  g2b_launch(seed_slots_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, 
      seq_state, words, slots, streams, n, (uint32_t)(seed & 0xffffffffull), (uint32_t)(seed >> 32));
  return g2b_check_launch("seed_slots");
}
