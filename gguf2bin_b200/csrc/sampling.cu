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
// r <= cumulative sum.  Implemented as weighted radix descents over the order-preserving
// integer image of the logits, so no sort of the vocabulary is needed.
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
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float *__restrict__ logits, int V, int ld, float temp, int *seq_state,
                   int state_words, const int *__restrict__ slots, int *__restrict__ out_ids) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  __shared__ float s_part[SAMPLE_THREADS];
  __shared__ int s_choice;
  const float *row = logits + (size_t)blockIdx.x * ld;
  if (temp <= 0.f) {
    const int id = block_argmax(row, V, 1.f, nullptr);
    if (threadIdx.x == 0) out_ids[blockIdx.x] = id;
    return;
  }
  float mx;
  block_argmax(row, V, 1.f, &mx);                  // max of the raw logits
  mx = mx / temp;
  // every thread owns a contiguous chunk so that the cumulative sum runs in index order
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int begin = min(V, (int)threadIdx.x * chunk), end = min(V, begin + chunk);
  float part = 0.f;
  for (int i = begin; i < end; ++i) part += expf(row[i] / temp - mx);
  s_part[threadIdx.x] = part;
  const float total = block_sum(part, scratch);
  __syncthreads();
  if (threadIdx.x == 0) {
    const float r = next_uniform(seq_state, slots[blockIdx.x], state_words);
    // first i with r <= c_i where c_i = (e_0 + ... + e_i) / total
    float c = 0.f;
    int owner = -1;
    for (int t = 0; t < (int)blockDim.x; ++t) {
      if (r <= (c + s_part[t]) / total && s_part[t] > 0.f) { owner = t; break; }
      c += s_part[t];
    }
    int choice = V - 1;
    if (owner >= 0) {
      const int b = min(V, owner * chunk), e = min(V, b + chunk);
      for (int i = b; i < e; ++i) {
        c += expf(row[i] / temp - mx);
        if (r <= c / total) { choice = i; break; }
        if (i == e - 1) choice = i;                // rounding: stay inside the owner's chunk
      }
    }
    s_choice = choice;
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
// `above + running weight` first reaches target; `*count_out` gets how many equal-key
// entries are taken (including it).  Sequential over the equal-key entries by thread 0:
// ties are rare.
template <bool MASS>
__device__ int tie_walk(const float *row, int V, float inv_temp, float mx, uint32_t key,
                        float above, float target, int *count_out) {
  __shared__ int s_idx, s_cnt;
  if (threadIdx.x == 0) {
    float run = above;
    int idx = -1, cnt = 0;
    for (int i = 0; i < V; ++i) {
      const float v = row[i] * inv_temp;
      if (order_key(v) != key) continue;
      run += MASS ? expf(v - mx) : 1.f;
      ++cnt;
      idx = i;
      if (run >= target) break;
    }
    s_idx = idx;
    s_cnt = cnt;
  }
  __syncthreads();
  const int idx = s_idx;
  if (count_out) *count_out = s_cnt;
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

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_filtered_kernel(float *__restrict__ logits, int V, int ld, float temp, int top_k,
                       float top_p, float penalty, const int *__restrict__ recent, int recent_ld,
                       const int *__restrict__ recent_n, int *seq_state, int state_words,
                       const int *__restrict__ slots, int *__restrict__ out_ids) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  __shared__ float hist[256];
  __shared__ float s_r;
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

  // kept set: key > bound_key, or key == bound_key with index <= tie_idx
  bool bounded = false;
  uint32_t bound_key = 0u;
  int tie_idx = V;
  if (top_k > 0 && top_k < V) {
    const Descent d = radix_descent<false>(row, V, inv_temp, mx, 0u, false, (float)top_k, hist);
    tie_idx = tie_walk<false>(row, V, inv_temp, mx, d.key, d.above, (float)top_k, nullptr);
    bound_key = d.key;
    bounded = true;
  }
  float kept = admitted_mass(row, V, inv_temp, mx, bound_key, tie_idx, bounded, scratch);
  if (top_p < 1.f) {
    // shortest prefix (descending) whose cumulative probability reaches top_p
    const float target = top_p * kept;
    const Descent d = radix_descent<true>(row, V, inv_temp, mx, bound_key, bounded, target, hist);
    int t2 = tie_walk<true>(row, V, inv_temp, mx, d.key, d.above, target, nullptr);
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
  int choice = tie_walk<true>(row, V, inv_temp, mx, d.key, d.above, target, nullptr);
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
