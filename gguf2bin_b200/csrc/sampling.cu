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
// (counting passes over the order-preserving integer image of the logits find where the
// k-th largest lies; a top_k of up to 64 over a large vocabulary is listed slice by slice by
// many blocks first); without a top_k the row is summed by buckets of its values, and only the
// buckets in which the cut and the draw fall are listed; weighted radix descents over the
// integer image do the same without any list when none fits (thousands of equal logits).
#include "common.cuh"

#include <climits>

G2B_DEFINE_LAST_ERROR

#ifndef SAMPLE_THREADS
#define SAMPLE_THREADS 1024
#endif

#ifdef G2B_SAMPLE_TIMING
// Development aid (off unless built with -DG2B_SAMPLE_TIMING): the clock of block (0, 0) at the ends
// of the phases of the filtered sampler's two kernels; g2b_sample_stamps copies them out.
__device__ long long g2b_stamps[32];
#define G2B_STAMP(i)                                                                      \
  do {                                                                                    \
    __syncthreads();                                                                      \
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) g2b_stamps[i] = clock64(); \
  } while (0)
extern "C" int g2b_sample_stamps(long long *out) {
  return cudaMemcpyFromSymbol(out, g2b_stamps, sizeof(g2b_stamps)) == cudaSuccess ? 0 : 1;
}
#else
#define G2B_STAMP(i) do { } while (0)
#endif

// Words of a sequence's record (seq_state[slot]): the sampler's key (seed, stream id), its draw
// counter, the count of tokens written to the ring of recent ids, and the ring itself.  The
// repeat penalty looks at the last RECENT_WINDOW ids; the ring is a few longer, so that the one
// step a decode session may take back leaves the window as it was.
constexpr int SS_DRAWS = 3, SS_RECENT_TOTAL = 4, SS_RING = 8, SS_RING_WORDS = 72;
constexpr int RECENT_WINDOW = 64;

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
  philox4x32_10((uint32_t)rec[SS_DRAWS], (uint32_t)rec[2], 0u, 0u, (uint32_t)rec[0], (uint32_t)rec[1], o);
  rec[SS_DRAWS] += 1;
  return (float)(o[0] >> 8) * (1.0f / 16777216.0f);
}

// Every entry of a row, once, by the threads of a block: f(index, value).  Four 16-byte loads
// per thread are in flight at a time when the row allows it (one block reading 4 bytes per
// thread and trip took 90 us for a vocabulary of 150k entries; this takes 6).
template <typename F>
__device__ __forceinline__ void scan_row(const float *__restrict__ row, int V, F f) {
  const int n4 = (((uintptr_t)row & 15) == 0) ? V / 4 : 0;
  const float4 *r4 = reinterpret_cast<const float4 *>(row);
  const int nt = blockDim.x;
  int i4 = threadIdx.x;
  for (; i4 + 3 * nt < n4; i4 += 4 * nt) {
    const float4 a = r4[i4], b = r4[i4 + nt], c = r4[i4 + 2 * nt], d = r4[i4 + 3 * nt];
    f(4 * i4, a.x); f(4 * i4 + 1, a.y); f(4 * i4 + 2, a.z); f(4 * i4 + 3, a.w);
    f(4 * (i4 + nt), b.x); f(4 * (i4 + nt) + 1, b.y); f(4 * (i4 + nt) + 2, b.z); f(4 * (i4 + nt) + 3, b.w);
    f(4 * (i4 + 2 * nt), c.x); f(4 * (i4 + 2 * nt) + 1, c.y); f(4 * (i4 + 2 * nt) + 2, c.z); f(4 * (i4 + 2 * nt) + 3, c.w);
    f(4 * (i4 + 3 * nt), d.x); f(4 * (i4 + 3 * nt) + 1, d.y); f(4 * (i4 + 3 * nt) + 2, d.z); f(4 * (i4 + 3 * nt) + 3, d.w);
  }
  for (; i4 < n4; i4 += nt) {
    const float4 a = r4[i4];
    f(4 * i4, a.x); f(4 * i4 + 1, a.y); f(4 * i4 + 2, a.z); f(4 * i4 + 3, a.w);
  }
  for (int i = 4 * n4 + threadIdx.x; i < V; i += nt) f(i, row[i]);
}

// ---- block argmax: lowest index among equal maxima ---------------------------
__device__ int block_argmax(const float *row, int V, float inv_temp, float *best_out) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  scan_row(row, V, [&](int i, float x) {
    const float v = x * inv_temp;
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  });
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
// Temperature: the row is cut into pieces of G consecutive entries (G = 128, or a multiple for
// rows beyond 262,144 entries), and one pass leaves the sum of e^(x/T - max) of every piece in
// shared memory: a warp takes a piece at a time, 128 entries per trip (16 bytes per lane).  The
// cumulative sum then runs in index order: over the pieces (32 lanes, a run of pieces each, and
// a prefix sum over the lanes) to the piece that holds the crossing, and inside that piece by a
// prefix sum over its entries.
constexpr int MAX_PIECES = 2048;
// Every thread of the block calls it; returns the chosen index to all of them.  s_piece:
// MAX_PIECES floats of shared memory.
__device__ int pick_by_temperature(const float *__restrict__ row, int V, float temp, float *s_piece,
                                   int *seq_state, int slot, int state_words,
                                   const float2 *__restrict__ pieces = nullptr) {
  __shared__ float s_before, s_target;
  __shared__ int s_owner, s_choice;
  __shared__ float s_wmax[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_warps = blockDim.x >> 5;
  const int trips = (V + 128 * MAX_PIECES - 1) / (128 * MAX_PIECES);     // trips of 128 entries per piece
  const int G = 128 * trips, n_pieces = (V + G - 1) / G;
  float mx;
  if (pieces) {                                    // max of x / temp over the pieces' maxima
    float m = -INFINITY;
    for (int j = threadIdx.x; j < n_pieces; j += blockDim.x) m = fmaxf(m, pieces[j].x);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) s_wmax[warp] = m;
    __syncthreads();
    m = lane < n_warps ? s_wmax[lane] : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    mx = m;
  } else {
    block_argmax(row, V, 1.f, &mx);                // max of the raw logits
    mx = mx / temp;
  }
  const bool vec = ((uintptr_t)row & 15) == 0;
  // the four entries of this lane in the trip that starts at entry i0 (0 beyond the row)
  auto four = [&](int i0, float (&e)[4]) {
    const int i = i0 + 4 * lane;
    if (vec && i + 3 < V) {
      const float4 x = *reinterpret_cast<const float4 *>(row + i);
      e[0] = expf(x.x / temp - mx); e[1] = expf(x.y / temp - mx);
      e[2] = expf(x.z / temp - mx); e[3] = expf(x.w / temp - mx);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) e[q] = i + q < V ? expf(row[i + q] / temp - mx) : 0.f;
    }
  };
  if (pieces) {                                    // a piece's sum was taken against its own maximum
    for (int j = threadIdx.x; j < n_pieces; j += blockDim.x) {
      const float2 p = pieces[j];
      s_piece[j] = p.y > 0.f ? p.y * expf(p.x - mx) : 0.f;
    }
  } else {
    for (int j = warp; j < n_pieces; j += n_warps) {
      float part = 0.f;
      for (int t = 0; t < trips; ++t) {
        float e[4];
        four(j * G + 128 * t, e);
        part += (e[0] + e[1]) + (e[2] + e[3]);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      if (lane == 0) s_piece[j] = part;
    }
  }
  __syncthreads();
  if (warp == 0) {
    // lane l owns the pieces [l per, (l + 1) per); first the lane, then the piece in it
    const int per = (n_pieces + 31) / 32;
    const int p0 = min(n_pieces, lane * per), p1 = min(n_pieces, p0 + per);
    float mine = 0.f;
    for (int j = p0; j < p1; ++j) mine += s_piece[j];
    float incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    const float total = __shfl_sync(0xffffffffu, incl, 31);
    float r = 0.f;
    if (lane == 0) r = next_uniform(seq_state, slot, state_words);
    r = __shfl_sync(0xffffffffu, r, 0);
    // first i with r <= c_i / total, taken as c_i >= r total
    const float target = r * total;
    const unsigned hit = __ballot_sync(0xffffffffu, mine > 0.f && incl >= target);
    if (hit) {
      const int l = __ffs(hit) - 1;
      const float c_l = __shfl_sync(0xffffffffu, incl - mine, l);
      if (lane == l) {
        float c = c_l;
        int j = p0;
        for (; j < p1; ++j) {
          if (s_piece[j] > 0.f && c + s_piece[j] >= target) break;
          c += s_piece[j];
        }
        if (j >= p1) {                               // rounding: the lane's last piece
          j = p1 - 1;
          c -= s_piece[j];
        }
        s_owner = j; s_before = c;
      }
    } else if (lane == 0) {
      s_owner = -1; s_before = 0.f;
    }
    if (lane == 0) s_target = target;
    __syncwarp();
    const int owner = s_owner;
    int choice = V - 1;
    if (owner >= 0) {
      float c = s_before;
      choice = min(V, (owner + 1) * G) - 1;          // rounding: stay inside the piece
      for (int t = 0; t < trips; ++t) {
        float e[4];
        const int i0 = owner * G + 128 * t;
        four(i0, e);
        const float mine4 = (e[0] + e[1]) + (e[2] + e[3]);
        float inc = mine4;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float up = __shfl_up_sync(0xffffffffu, inc, o);
          if (lane >= o) inc += up;
        }
        float run = c + inc - mine4;                 // before this lane's four
        int found = -1;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          run += e[q];
          if (found < 0 && i0 + 4 * lane + q < V && run >= s_target) found = i0 + 4 * lane + q;
        }
        const unsigned any = __ballot_sync(0xffffffffu, found >= 0);
        if (any) {
          choice = __shfl_sync(0xffffffffu, found, __ffs(any) - 1);
          break;
        }
        c += __shfl_sync(0xffffffffu, inc, 31);
      }
    }
    if (lane == 0) s_choice = choice;
  }
  __syncthreads();
  return s_choice;
}

// The pieces' sums by many blocks per row: a warp per piece, which leaves the piece's maximum of
// x / temp and its sum of e^(x/temp - that maximum) in pieces[row][piece]; the row's block then
// scales each sum to the row's maximum instead of reading the row (twice) itself: 38 us by one
// block for 150k entries.
constexpr int PIECE_BLOCKS = 64, PIECE_THREADS = 256;

__global__ void __launch_bounds__(PIECE_THREADS)
temperature_pieces_kernel(const float *__restrict__ logits, int V, int ld, float temp, float2 *__restrict__ pieces) {
  pdl_launch();
  pdl_wait();
  const float *row = logits + (size_t)blockIdx.y * ld;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int trips = (V + 128 * MAX_PIECES - 1) / (128 * MAX_PIECES);
  const int G = 128 * trips, n_pieces = (V + G - 1) / G;
  const bool vec = ((uintptr_t)row & 15) == 0;
  float2 *out = pieces + (size_t)blockIdx.y * MAX_PIECES;
  for (int j = blockIdx.x * (PIECE_THREADS / 32) + warp; j < n_pieces; j += PIECE_BLOCKS * (PIECE_THREADS / 32)) {
    float m = -INFINITY, sum = 0.f;                // running maximum and sum against it, trip by trip
    for (int t = 0; t < trips; ++t) {
      const int i = j * G + 128 * t + 4 * lane;
      float x[4];
      if (vec && i + 3 < V) {
        const float4 v = *reinterpret_cast<const float4 *>(row + i);
        x[0] = v.x / temp; x[1] = v.y / temp; x[2] = v.z / temp; x[3] = v.w / temp;
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) x[q] = i + q < V ? row[i + q] / temp : -INFINITY;
      }
      float tm = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
      if (tm == -INFINITY) continue;               // nothing of the row in this trip
      const float m_new = fmaxf(m, tm);
      float part = 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) part += x[q] == -INFINITY ? 0.f : expf(x[q] - m_new);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      sum = (m == -INFINITY ? 0.f : sum * expf(m - m_new)) + part;
      m = m_new;
    }
    if (lane == 0) out[j] = make_float2(m, sum);
  }
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float *__restrict__ logits, int V, int ld, float temp, int *seq_state,
                   int state_words, const int *__restrict__ slots, int *__restrict__ out_ids,
                   const float2 *__restrict__ pieces) {
  pdl_launch();
  pdl_wait();
  __shared__ float s_piece[MAX_PIECES];
  const float *row = logits + (size_t)blockIdx.x * ld;
  const int id = temp <= 0.f ? block_argmax(row, V, 1.f, nullptr)
                             : pick_by_temperature(row, V, temp, s_piece, seq_state, slots[blockIdx.x], state_words,
                                                   pieces ? pieces + (size_t)blockIdx.x * MAX_PIECES : nullptr);
  if (threadIdx.x == 0) out_ids[blockIdx.x] = id;
}

// pieces: scratch of R x 2,048 x 2 floats, or null; with it, the pieces' sums of a large
// vocabulary are taken by many blocks per row first (temperature_pieces_kernel).
extern "C" int g2b_sample_rows(const float *logits, int R, int V, int ld, float temp,
                               int *seq_state, int state_words, const int *slots, int *out_ids,
                               float *pieces, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || ld < V) G2B_REFUSE("sample_rows: bad sizes V=%d ld=%d", V, ld);
  if (temp > 0.f && (!seq_state || !slots || state_words < 4))
    G2B_REFUSE("sample_rows: temperature sampling needs the per-slot state");
  const bool split = pieces && temp > 0.f && V >= 8192 && R <= 65535 && (((uintptr_t)pieces) & 7) == 0;
  if (split) {
    g2b_launch(temperature_pieces_kernel, dim3(PIECE_BLOCKS, R), dim3(PIECE_THREADS), 0, stream, logits, V, ld,
               temp, (float2 *)pieces);
    int rc = g2b_check_launch("sample_rows (pieces)");
    if (rc) return rc;
  }
  g2b_launch(sample_rows_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream, logits, V, ld, temp, seq_state,
             state_words, slots, out_ids, (const float2 *)(split ? pieces : nullptr));
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
    scan_row(row, V, [&](int, float x) {
      const float v = x * inv_temp;
      const uint32_t k = order_key(v);
      if (bounded && k < bound_key) return;        // below the kept set
      if ((k & mask) != (prefix & mask)) return;
      const float w = MASS ? expf(v - mx) : 1.f;
      atomicAdd(&hist[(k >> shift) & 0xffu], w);
    });
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
  scan_row(row, V, [&](int i, float x) {
    if (order_key(x * inv_temp) == key) {
      const int j = atomicAdd(&s_n, 1);
      if (j < TIE_CAP) tie_list[j] = i;
    }
  });
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
  scan_row(row, V, [&](int i, float x) {
    const float v = x * inv_temp;
    const uint32_t k = order_key(v);
    if (bounded && (k < bound_key || (k == bound_key && i > tie_idx))) return;
    part += expf(v - mx);
  });
  return block_sum(part, scratch);
}

// ---- the kept entries as a short list ---------------------------------------------------
// With a top_k of a few dozen, or a top_p that a few hundred entries reach, the kept set is
// tiny: every entry at or above a 22-bit prefix of the key is listed (a complete head of the
// row's descending order), the list is sorted (key descending, then index ascending: the
// reference's order), and the cuts and the draw are walks over it.  The prefix comes from a
// look at 4,096 entries of the row, or, when that guess fails, from two counting passes over
// the whole row.  When neither gives a list that fits (thousands of logits sharing 22 bits, a
// top_p that needs more than the list holds) the caller takes the descents over the whole row.
constexpr int LIST_CAP = 2048;
struct ShortList {
  uint32_t key[LIST_CAP];
  int idx[LIST_CAP];
  float e[LIST_CAP];
  int hist[2048];
};

// From the top bin down to the one where the running count reaches `want`: lane l of warp 0 owns
// the 64 bins below 2048 - 64 l; a prefix sum over the lanes finds the lane, which walks its
// own bins.  *chosen: that bin (the lowest one if the count is never reached); *above: the
// count in the bins above it.  Warp 0 calls it; the others skip it.
__device__ __forceinline__ void walk_bins(const int *hist, int above0, int want, int *chosen_out, int *above_out) {
  const int lane = threadIdx.x & 31, hi = 2047 - 64 * lane;
  int mine = 0;
  // (the lanes' ranges lie 64 words apart, all in one bank: each lane starts at another place of its range)
  for (int d = 0; d < 64; ++d) mine += hist[hi - ((d + lane) & 63)];
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  const unsigned hit = __ballot_sync(0xffffffffu, above0 + incl >= want);
  const int owner = hit ? __ffs(hit) - 1 : 31;
  // the owner's 64 bins by all lanes, two each, from the top down
  const int top = 2047 - 64 * owner;
  const int before = __shfl_sync(0xffffffffu, above0 + incl - mine, owner);      // count above the owner's bins
  const int h0 = hist[top - 2 * lane], h1 = hist[top - 2 * lane - 1];
  int pair = h0 + h1;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, pair, o);
    if (lane >= o) pair += up;
  }
  const int c0 = before + pair - h1, c1 = before + pair;       // counts down to and including bin top - 2 lane, top - 2 lane - 1
  const unsigned r0 = __ballot_sync(0xffffffffu, c0 >= want), r1 = __ballot_sync(0xffffffffu, c1 >= want);
  int chosen, above;
  if (r0 | r1) {
    const int l0 = r0 ? __ffs(r0) - 1 : 32, l1 = r1 ? __ffs(r1) - 1 : 32;
    const bool first = l0 <= l1;                     // the upper bin of lane l0 comes before the lower bin of lane l1 >= l0
    const int l = first ? l0 : l1;
    chosen = top - 2 * l - (first ? 0 : 1);
    above = __shfl_sync(0xffffffffu, first ? c0 - h0 : c1 - h1, l);
  } else {                                           // the count is never reached: the lowest bin
    chosen = top - 63;
    above = __shfl_sync(0xffffffffu, c1 - h1, 31);
  }
  *chosen_out = chosen;
  *above_out = above;
}

// Sorts the first n entries of the list: key descending, then index ascending.
__device__ void sort_list(ShortList &L, int n) {
  int n2 = 1;
  while (n2 < n) n2 <<= 1;
  for (int i = n + threadIdx.x; i < n2; i += blockDim.x) { L.key[i] = 0u; L.idx[i] = 0x7fffffff; }
  __syncthreads();
  for (int k = 2; k <= n2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < n2; i += blockDim.x) {
        const int p = i ^ j;
        if (p > i) {
          const bool up = (i & k) == 0;             // this pair in list order
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
}

// Sorts a list of up to RANK_SORT_MAX entries by counting, for every entry, the entries that belong
// before it: no barriers but two, where the bitonic network has one per step (21 steps for 64
// entries cost 2.8 us).  The sorted list passes through the list's other two arrays.
constexpr int RANK_SORT_MAX = 256;
__device__ void rank_sort(ShortList &L, int n) {
  uint32_t *tkey = reinterpret_cast<uint32_t *>(L.e);
  int *tidx = L.hist;
  __syncthreads();
  // four threads share an entry: each counts over a quarter of the list
  const int per_trip = blockDim.x >> 2, q = threadIdx.x & 3;
  for (int base = 0; base < n; base += per_trip) {
    const int i = base + (threadIdx.x >> 2);
    const bool live = i < n;
    const uint32_t k = live ? L.key[i] : 0u;
    const int id = live ? L.idx[i] : 0;
    int before = 0;
    if (live) {
#pragma unroll 4
      for (int j = q; j < n; j += 4) {
        const uint32_t kj = L.key[j];
        before += (kj > k || (kj == k && L.idx[j] < id)) ? 1 : 0;
      }
    }
    before += __shfl_xor_sync(0xffffffffu, before, 1);
    before += __shfl_xor_sync(0xffffffffu, before, 2);
    if (live && q == 0) {
      tkey[before] = k;
      tidx[before] = id;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) { L.key[i] = tkey[i]; L.idx[i] = tidx[i]; }
  __syncthreads();
}

// Every entry whose key has at least the 22-bit prefix `floor22` into the list; returns their
// number (which may exceed LIST_CAP: then the list is not complete).
__device__ int list_from_floor(const float *row, int V, float inv_temp, uint32_t floor22, ShortList &L) {
  __shared__ int s_n;
  __syncthreads();
  if (threadIdx.x == 0) s_n = 0;
  __syncthreads();
  scan_row(row, V, [&](int i, float x) {
    const uint32_t k = order_key(x * inv_temp);
    if ((k >> 10) >= floor22) {
      const int j = atomicAdd(&s_n, 1);
      if (j < LIST_CAP) { L.key[j] = k; L.idx[j] = i; }
    }
  });
  __syncthreads();
  return s_n;
}

// The `want` largest entries (and a few hundred more) in ONE pass over the row: 4,096 evenly
// spaced entries are looked at first, and the 22-bit prefix of the m-th largest of them, m a
// little more than want's share of the sample, is the floor of the list.  Returns the number of
// listed entries (sorted; a complete head of the row's descending order), or -1 when the floor
// turned out too high or too low (fewer than want entries, or more than the list holds): the
// caller then counts over the whole row.
__device__ int list_by_sampled_floor(const float *row, int V, float inv_temp, int want, ShortList &L) {
  __shared__ uint32_t s_prefix;
  __shared__ int s_above;
  constexpr int SAMPLES = 4096;
  static_assert(2 * LIST_CAP == SAMPLES, "the sample lives in the list's key and index arrays");
  uint32_t *samp = L.key;                           // key[] and idx[] are adjacent: 4,096 words
  const int S = min(V, SAMPLES);
  // three times want's share of the sample for a small want, one and a half for a large one, and 8
  const long long m64 = (long long)want * S * (want <= 128 ? 6 : 3) / (2LL * V) + 8;
  if (m64 > S / 2) return -1;                       // want is a large share of the row: count instead
  const int m = (int)m64;
  for (int t = threadIdx.x; t < S; t += blockDim.x)
    samp[t] = order_key(row[(long long)t * V / S] * inv_temp);
  if (threadIdx.x == 0) { s_prefix = 0u; s_above = 0; }
  __syncthreads();
  for (int pass = 0; pass < 2; ++pass) {
    const int shift = pass == 0 ? 21 : 10;
    for (int i = threadIdx.x; i < 2048; i += blockDim.x) L.hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    for (int t = threadIdx.x; t < S; t += blockDim.x) {
      const uint32_t k = samp[t];
      if (pass == 1 && (k >> 21) != (prefix >> 21)) continue;
      atomicAdd(&L.hist[(k >> shift) & 0x7ffu], 1);
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      int chosen, above;
      walk_bins(L.hist, s_above, m, &chosen, &above);
      if (threadIdx.x == 0) {
        s_above = above;
        s_prefix = prefix | ((uint32_t)chosen << shift);
      }
    }
    __syncthreads();
  }
  const uint32_t floor22 = s_prefix >> 10;
  const int n = list_from_floor(row, V, inv_temp, floor22, L);
  if (n < want || n > LIST_CAP) return -1;
  if (n <= RANK_SORT_MAX) rank_sort(L, n);
  else sort_list(L, n);
  return n;
}

// The same by counting: a pass over the row counts the keys by their upper 11 bits and finds the
// bin in which the want-th largest lies; if that bin and those above hold few entries they are the
// list, otherwise a second pass over the next 11 bits narrows the bin down.  (The counts are plain
// shared-memory additions: gathering a warp's equal bins first with match.any cost 1,300 cycles per
// entry where the bins differ.)  The last pass lists the entries at or above the floor.  -1 when
// more than the list holds share the 22-bit prefix.
__device__ int list_top_k(const float *row, int V, float inv_temp, int top_k, ShortList &L) {
  __shared__ uint32_t s_prefix;
  __shared__ int s_above, s_total;
  __syncthreads();
  if (threadIdx.x == 0) { s_prefix = 0u; s_above = 0; s_total = 0; }
  __syncthreads();
  for (int pass = 0; pass < 2; ++pass) {
    const int shift = pass == 0 ? 21 : 10;
    for (int i = threadIdx.x; i < 2048; i += blockDim.x) L.hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    scan_row(row, V, [&](int, float x) {
      const uint32_t k = order_key(x * inv_temp);
      if (pass == 1 && (k >> 21) != (prefix >> 21)) return;
      atomicAdd(&L.hist[(k >> shift) & 0x7ffu], 1);
    });
    __syncthreads();
    if (threadIdx.x < 32) {
      int chosen, above;
      walk_bins(L.hist, s_above, top_k, &chosen, &above);
      if (threadIdx.x == 0) {
        s_above = above;
        s_prefix = prefix | ((uint32_t)chosen << shift);
        s_total = above + L.hist[chosen];           // entries at or above the prefix so far
      }
    }
    __syncthreads();
    if (pass == 0 && s_total <= RANK_SORT_MAX) break;       // few enough: the bin's lower edge is the floor
  }
  const int total = s_total;
  G2B_STAMP(2);
  if (total > LIST_CAP || total < top_k) return -1;
  const int n = list_from_floor(row, V, inv_temp, s_prefix >> 10, L);
  G2B_STAMP(3);
  if (n > LIST_CAP) return -1;
  if (n <= RANK_SORT_MAX) rank_sort(L, n);
  else sort_list(L, n);
  G2B_STAMP(4);
  return n;
}

// Repeat penalty, each distinct id once (src/main.c:204-223), on the entries [begin, end) of the
// row: over the n ids the caller gives, or (ids == nullptr) over the last RECENT_WINDOW ids in the
// sequence's own ring `rec`.  Every thread of the block calls it.
__device__ void apply_penalty(float *row, int V, int begin, int end, float penalty, const int *ids, int n_ids,
                              const int *rec) {
  if (penalty == 1.f || (!ids && !rec)) return;
  const bool ring = ids == nullptr;
  const int *rc = ring ? rec + SS_RING : ids;
  const int total = ring ? max(rec[SS_RECENT_TOTAL], 0) : 0;
  const int n = ring ? min(total, RECENT_WINDOW) : n_ids;
  // entry i of the window (any order will do: every distinct id counts once)
  auto entry = [&](int i) { return ring ? rc[(total - 1 - i) % SS_RING_WORDS] : rc[i]; };
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int id = entry(i);
    if (id < begin || id >= end || id >= V) continue;
    bool first = true;
    for (int j = 0; j < i; ++j) if (entry(j) == id) { first = false; break; }
    if (!first) continue;
    const float v = row[id];
    row[id] = v > 0.f ? v / penalty : v * penalty;
  }
}

// ---- the best top_k of a row by many blocks ------------------------------------------------
// A row is one block's work above, and a block pulls a vocabulary of 150k entries through one SM
// at a few dozen GB/s: 50 us for the reference's default parameters.  With a top_k of up to
// MAX_SLICE_CAP the row is cut into slices first (32 for a top_k up to 64, 16 up to 128, 8 up to
// 256: their lists side by side are 2,048 places); a block per slice applies the repeat
// penalty to its entries and lists its own best top_k (sorted; every entry of the row's best
// top_k is among some slice's).  The row's block then merges the slices' lists instead
// of reading the row.  cand: int [rows x ROW_CAND_WORDS]: per row the slices' numbers of listed
// entries (-1: the slice's list did not fit, the row's block reads the row itself), the
// keys, the indices.
constexpr int MAX_SLICES = 32, FILTER_THREADS = 256;
constexpr int MAX_SLICE_CAP = 256;       // places per slice: 64 for a top_k up to 64 (32 slices), 128 (16), 256 (8)
constexpr int ROW_CAND_WORDS = MAX_SLICES + 2 * 2048;       // per row: the slices' counts, their keys, their indices

__host__ __device__ inline int slice_cap(int top_k) { return top_k <= 64 ? 64 : (top_k <= 128 ? 128 : 256); }

__global__ void __launch_bounds__(FILTER_THREADS)
filter_slices_kernel(float *__restrict__ logits, int V, int ld, float temp, int top_k, float penalty,
                     const int *__restrict__ recent, int recent_ld, const int *__restrict__ recent_n,
                     const int *seq_state, int state_words, const int *__restrict__ slots, int *__restrict__ cand) {
  pdl_launch();
  pdl_wait();
  __shared__ ShortList L;
  const int r = blockIdx.y;
  float *row = logits + (size_t)r * ld;
  const int cap = slice_cap(top_k), lists = 2048 / cap;
  // gridDim.x slices (as many as there are lists with few rows, fewer with many: enough blocks to
  // fill the GPU once); the places of the others are marked empty
  const int per = ((V + (int)gridDim.x - 1) / (int)gridDim.x + 3) & ~3;     // slices start at multiples of 16 bytes
  const int begin = min(V, (int)blockIdx.x * per), end = min(V, begin + per);
  int *mine = cand + (size_t)r * ROW_CAND_WORDS;
  if (blockIdx.x == 0)
    for (int sl = gridDim.x + threadIdx.x; sl < lists; sl += blockDim.x) mine[sl] = 0;
  const int *rec = (seq_state && slots && state_words >= SS_RING + SS_RING_WORDS)
                       ? seq_state + (size_t)slots[r] * state_words : nullptr;
  G2B_STAMP(0);
  apply_penalty(row, V, begin, end, penalty, recent ? recent + (size_t)r * recent_ld : nullptr,
                recent ? min(max(recent_n[r], 0), recent_ld) : 0, rec);
  __syncthreads();
  G2B_STAMP(1);
  const int want = min(top_k, end - begin);
  int n = 0;
  if (want > 0) n = list_top_k(row + begin, end - begin, 1.f / temp, want, L);
  const int m = n < 0 ? -1 : min(n, want);
  int *keys = mine + MAX_SLICES + blockIdx.x * cap, *idxs = keys + 2048;
  for (int j = threadIdx.x; j < m; j += blockDim.x) {
    keys[j] = (int)L.key[j];
    idxs[j] = begin + L.idx[j];
  }
  if (threadIdx.x == 0) mine[blockIdx.x] = m;
  G2B_STAMP(5);
}

// How many entries of the sorted list (zk, zi)[0, n), n <= cap (a power of two), belong before the
// entry (k, id): a search without branches, the same steps for every lane.
__device__ __forceinline__ int count_before(const uint32_t *zk, const int *zi, int n, int cap, uint32_t k, int id) {
  int pos = 0;
  for (int step = cap; step > 0; step >>= 1) {
    const int m = pos + step;                        // are the first m entries all before (k, id)?
    const int at = min(m, n) - 1;
    const uint32_t mk = zk[max(at, 0)];
    const int mi = zi[max(at, 0)];
    const bool before = m <= n && (mk > k || (mk == k && mi < id));
    pos = before ? m : pos;
  }
  return pos;
}

// The best `want` entries of a row from its slices' sorted lists: the lists are merged in pairs,
// level by level, each result cut to `want`; an entry's place in a merged list is its place in its own
// list plus the number of entries of the other list that belong before it (a binary search), so a
// level is one step for all entries at once.  cand: the row's part of the scratch; cap: places per
// list (2,048 / cap lists).  -1 when a slice gave no list.
__device__ int list_from_slices(const int *__restrict__ cand, int cap, int want, ShortList &L) {
  static_assert(LIST_CAP == 2048, "the lists side by side fill the list's arrays");
  __shared__ int s_len[2][MAX_SLICES];
  uint32_t *ik = L.key, *ok = reinterpret_cast<uint32_t *>(L.e);      // this level's lists, the next level's
  int *ii = L.idx, *oi = L.hist;
  const int shift = cap == 64 ? 6 : (cap == 128 ? 7 : 8);     // cap is 64, 128 or 256
  const int lists0 = LIST_CAP >> shift;
  __syncthreads();
  if (threadIdx.x < MAX_SLICES) s_len[0][threadIdx.x] = threadIdx.x < lists0 ? cand[threadIdx.x] : 0;
  __syncthreads();
  G2B_STAMP(12);
  const int my_len = s_len[0][threadIdx.x & 31];      // every warp looks at all the lengths
  if (__any_sync(0xffffffffu, my_len < 0 || my_len > cap)) return -1;
  for (int t = threadIdx.x; t < LIST_CAP; t += blockDim.x) {
    if ((t & (cap - 1)) < s_len[0][t >> shift]) {
      L.key[t] = (uint32_t)cand[MAX_SLICES + t];
      L.idx[t] = cand[MAX_SLICES + LIST_CAP + t];
    }
  }
  __syncthreads();
  G2B_STAMP(13);
  int from = 0;
  for (int lists = lists0; lists > 1; lists >>= 1, from ^= 1) {
    for (int t = threadIdx.x; t < (lists << shift); t += blockDim.x) {
      const int mine = t >> shift, j = t & (cap - 1), other = mine ^ 1;
      if (j < s_len[from][mine]) {
        const uint32_t k = ik[t];
        const int id = ii[t];
        const int place = j + count_before(ik + (other << shift), ii + (other << shift), s_len[from][other], cap, k, id);
        if (place < want) {
          ok[((mine >> 1) << shift) + place] = k;
          oi[((mine >> 1) << shift) + place] = id;
        }
      }
    }
    if (threadIdx.x < lists / 2)
      s_len[from ^ 1][threadIdx.x] = min(want, s_len[from][2 * threadIdx.x] + s_len[from][2 * threadIdx.x + 1]);
    __syncthreads();
    uint32_t *tk = ik; ik = ok; ok = tk;
    int *ti = ii; ii = oi; oi = ti;
  }
  G2B_STAMP(14);
  const int n = s_len[from][0];
  if (from == 1) {                                   // (an odd number of levels: the result is in the second pair of arrays)
    for (int i = threadIdx.x; i < n; i += blockDim.x) { L.key[i] = ik[i]; L.idx[i] = ii[i]; }
    __syncthreads();
  }
  return n;
}

// ---- without a top_k: the row by buckets of its values ------------------------------------------
// A top_p alone (or nothing but the repeat penalty) keeps whatever share of the vocabulary holds the
// mass: a few entries of a peaked distribution, tens of thousands of a flat one, which no short
// list holds; finding the cut by radix descents over the keys took 1.5 ms for 150k entries (every
// pass adds 150k weights into a handful of bins).  Here one pass adds every entry's e^(v - max)
// and a count into the bucket floor(64 (max - v)) of its value v = x / temp (2,048 buckets: 32
// units below the maximum, what lies further down shares the last one).  Buckets are in descending
// order of value, so the cumulative sums over them say in which bucket the top_p cut falls and in
// which the draw; only those one or two buckets are listed, sorted (key descending, index
// ascending: the reference's order) and walked.  Returns the chosen index to every thread, or -1
// when a bucket that has to be listed holds more than the list does (the caller's descents then).
// Warp 0 calls it: the first j < n with base + e[0] + ... + e[j] >= target (n if there is none) and
// that sum (the whole sum if there is none).
__device__ int first_reaching(const float *e, int n, float base, float target, float *sum_out) {
  const int lane = threadIdx.x & 31;
  float run = base;
  for (int i0 = 0; i0 < n; i0 += 32) {
    const float x = i0 + lane < n ? e[i0 + lane] : 0.f;
    float incl = x;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    const unsigned hit = __ballot_sync(0xffffffffu, i0 + lane < n && run + incl >= target);
    if (hit) {
      const int l = __ffs(hit) - 1;
      *sum_out = run + __shfl_sync(0xffffffffu, incl, l);
      return i0 + l;
    }
    run += __shfl_sync(0xffffffffu, incl, 31);
  }
  *sum_out = run;
  return n;
}

constexpr int N_BUCKETS = 2048;
constexpr float BUCKETS_PER_UNIT = 64.f;
__device__ __forceinline__ int bucket_of(float v, float mx) {
  return max(0, min(N_BUCKETS - 1, (int)((mx - v) * BUCKETS_PER_UNIT)));     // falls as v rises; the maximum is in bucket 0
}

// The entries of bucket b into the list, sorted, with their weights in le; their number.
__device__ int list_bucket(const float *row, int V, float inv_temp, float mx, int b, ShortList &L, float *le) {
  __shared__ int s_n;
  __syncthreads();
  if (threadIdx.x == 0) s_n = 0;
  __syncthreads();
  scan_row(row, V, [&](int i, float x) {
    const float v = x * inv_temp;
    if (bucket_of(v, mx) == b) {
      const int j = atomicAdd(&s_n, 1);
      if (j < LIST_CAP) { L.key[j] = order_key(v); L.idx[j] = i; }
    }
  });
  __syncthreads();
  const int n = s_n;
  if (n > LIST_CAP) return n;
  sort_list(L, n);                                   // in place: the list's other arrays hold the buckets
  for (int j = threadIdx.x; j < n; j += blockDim.x) le[j] = expf(row[L.idx[j]] * inv_temp - mx);
  __syncthreads();
  return n;
}

__device__ int pick_by_buckets(const float *row, int V, float inv_temp, float top_p, float u, ShortList &L, float *le) {
  static_assert(N_BUCKETS == 2048 && LIST_CAP == 2048, "the buckets live in the list's arrays");
  __shared__ int s_keep, s_choice;
  __shared__ float s_kept, s_base;
  float *mass = L.e;                                 // per bucket, then cumulative from the top
  int *cnt = L.hist;
  float mx;
  block_argmax(row, V, inv_temp, &mx);
  for (int i = threadIdx.x; i < N_BUCKETS; i += blockDim.x) { mass[i] = 0.f; cnt[i] = 0; }
  __syncthreads();
  scan_row(row, V, [&](int, float x) {
    const float v = x * inv_temp;
    const int b = bucket_of(v, mx);
    atomicAdd(&mass[b], expf(v - mx));
    atomicAdd(&cnt[b], 1);
  });
  __syncthreads();
  if (threadIdx.x < 32) {
    // cumulative sums in bucket order: lane l owns the 64 buckets from 64 l
    const int lane = threadIdx.x, b0 = 64 * lane;
    float mine = 0.f;
    for (int d = 0; d < 64; ++d) mine += mass[b0 + d];
    float incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    float run = incl - mine;
    for (int d = 0; d < 64; ++d) { run += mass[b0 + d]; mass[b0 + d] = run; }
  }
  __syncthreads();
  // first bucket, up to b_max, whose cumulative sum reaches target (b_max if none does)
  auto bucket_reaching = [&](float target, int b_max) {
    int lo = 0, hi = b_max;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (mass[mid] >= target) hi = mid; else lo = mid + 1;
    }
    while (lo > 0 && cnt[lo] == 0) --lo;             // (rounding left the target above the total: the last entries)
    return lo;
  };
  const float total = mass[N_BUCKETS - 1];
  int bp = N_BUCKETS - 1, n_p = 0;                   // the cut's bucket and the entries listed from it
  if (top_p < 1.f) {
    const float target = top_p * total;
    bp = bucket_reaching(target, N_BUCKETS - 1);
    if (cnt[bp] > LIST_CAP) return -1;
    const float base = bp > 0 ? mass[bp - 1] : 0.f;
    n_p = list_bucket(row, V, inv_temp, mx, bp, L, le);
    if (threadIdx.x < 32) {
      float kept;
      const int j = first_reaching(le, n_p, base, target, &kept);       // the shortest head that reaches top_p
      if (threadIdx.x == 0) { s_keep = j < n_p ? j + 1 : n_p; s_kept = kept; s_base = base; }
    }
    __syncthreads();
  } else if (threadIdx.x == 0) {
    s_kept = total; s_keep = 0; s_base = 0.f;
  }
  __syncthreads();
  const float kept = s_kept, target = u * kept;
  const int keep_p = s_keep;
  int bu = bucket_reaching(target, bp);
  // (with a cut, the draw falls in the cut's bucket when it lies beyond the buckets above it)
  if (top_p < 1.f && target > s_base) bu = bp;
  int n_u = n_p, limit = keep_p;
  float base = s_base;
  if (!(top_p < 1.f && bu == bp)) {
    if (cnt[bu] > LIST_CAP) return -1;
    base = bu > 0 ? mass[bu - 1] : 0.f;
    n_u = list_bucket(row, V, inv_temp, mx, bu, L, le);
    limit = n_u;
  }
  if (threadIdx.x < 32) {
    float sum;
    const int j = first_reaching(le, limit, base, target, &sum);
    if (threadIdx.x == 0) s_choice = L.idx[limit > 0 ? min(j, limit - 1) : 0];
  }
  __syncthreads();
  (void)n_u;
  return s_choice;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_filtered_kernel(float *__restrict__ logits, int V, int ld, float temp, int top_k,
                       float top_p, float penalty, const int *__restrict__ recent, int recent_ld,
                       const int *__restrict__ recent_n, int *seq_state, int state_words,
                       const int *__restrict__ slots, int *__restrict__ out_ids, int append,
                       const int *__restrict__ cand_all) {
  pdl_launch();
  pdl_wait();
  const int *cand = cand_all ? cand_all + (size_t)blockIdx.x * ROW_CAND_WORDS : nullptr;
  G2B_STAMP(8);
  __shared__ float scratch[32];
  __shared__ float s_r;
  __shared__ int s_done;
  __shared__ ShortList L;
  __shared__ float s_le[LIST_CAP];
  float *hist = L.e;                                // the descents' 256 bins and the tie list live in the list's arrays
  int *tie_list = L.idx;
  float *row = logits + (size_t)blockIdx.x * ld;

  int *rec = (seq_state && slots && state_words >= SS_RING + SS_RING_WORDS)
                 ? seq_state + (size_t)slots[blockIdx.x] * state_words : nullptr;
  const bool ring = recent == nullptr && rec != nullptr;
  if (!cand) {                                      // (with candidates, the kernel that listed them has done it)
    apply_penalty(row, V, 0, V, penalty, recent ? recent + (size_t)blockIdx.x * recent_ld : nullptr,
                  recent ? min(max(recent_n[blockIdx.x], 0), recent_ld) : 0, rec);
    __syncthreads();
  }
  // the chosen id goes into the ring (a caller that keeps the recent ids itself passes them in)
  auto keep = [&](int id) {
    out_ids[blockIdx.x] = id;
    if (ring && append) {
      const int total = max(rec[SS_RECENT_TOTAL], 0);
      rec[SS_RING + total % SS_RING_WORDS] = id;
      rec[SS_RECENT_TOTAL] = total + 1;
    }
  };
  if (temp <= 0.f) {
    const int id = block_argmax(row, V, 1.f, nullptr);
    if (threadIdx.x == 0) keep(id);
    return;
  }
  const float inv_temp = 1.f / temp;
  float mx;
  const bool cut_k = top_k > 0 && top_k < V;
  // The token's one random number, whichever way the kept set is found below.  Thread 0 asks for the
  // record's words here and computes the number where it is first needed: two dependent trips to
  // memory that would otherwise stand before the block's first barrier.
  uint32_t draw_words[4] = {0u, 0u, 0u, 0u};
  int *draw_rec = nullptr;
  if (threadIdx.x == 0) {
    draw_rec = seq_state + (size_t)slots[blockIdx.x] * state_words;
    draw_words[0] = (uint32_t)draw_rec[SS_DRAWS]; draw_words[1] = (uint32_t)draw_rec[2];
    draw_words[2] = (uint32_t)draw_rec[0]; draw_words[3] = (uint32_t)draw_rec[1];
  }
  bool drawn = false;
  float u = 0.f;
  // every thread calls it, once is enough: the number to all threads (a barrier inside)
  auto draw = [&]() {
    if (drawn) return;
    if (threadIdx.x == 0) {
      uint32_t o[4];
      philox4x32_10(draw_words[0], draw_words[1], 0u, 0u, draw_words[2], draw_words[3], o);
      draw_rec[SS_DRAWS] = (int)draw_words[0] + 1;
      s_r = (float)(o[0] >> 8) * (1.0f / 16777216.0f);
    }
    __syncthreads();
    u = s_r;
    drawn = true;
  };
  if (!cut_k) {
    draw();
    // no top_k: the row by buckets of its values (a flat distribution keeps tens of thousands of entries)
    const int id = pick_by_buckets(row, V, inv_temp, top_p, u, L, s_le);
    if (id >= 0) {
      if (threadIdx.x == 0) keep(id);
      return;
    }
  }
  // (When nothing is cut, the draw still walks the entries in descending order, as the
  // reference's filtered sampler does: the descents below.)
  // The kept entries as a sorted list: the best top_k, or without a top_k the best 512 or more, among
  // which the shortest head that reaches top_p of the WHOLE row's mass usually lies.
  const int want = cut_k ? top_k : min(V, 512);
  if (want <= LIST_CAP && (cut_k || top_p < 1.f)) {
    int n = cand ? list_from_slices(cand, slice_cap(top_k), want, L) : list_by_sampled_floor(row, V, inv_temp, want, L);
    G2B_STAMP(9);
    if (n < 0 && cut_k) n = list_top_k(row, V, inv_temp, top_k, L);
    if (n >= 0) {
      const int n_list = cut_k ? min(n, top_k) : n;
      mx = row[L.idx[0]] * inv_temp;               // the list's head is the row's maximum
      float whole = 0.f;                            // without a top_k: the mass of the whole row
      if (!cut_k) whole = admitted_mass(row, V, inv_temp, mx, 0u, V, false, scratch);
      for (int j = threadIdx.x; j < n_list; j += blockDim.x) L.e[j] = expf(row[L.idx[j]] * inv_temp - mx);
      __syncthreads();
      draw();
      G2B_STAMP(10);
      if (cut_k && n_list >= 1) {
        // a top_k's list: the cumulative sums by one warp, 32 entries a trip (the cuts and the draw by
        // one thread walking the list took 3 us for 40 entries)
        if (threadIdx.x < 32) {
          const int lane = threadIdx.x;
          float run = 0.f;                           // the weights become their cumulative sums, in place
          for (int i0 = 0; i0 < n_list; i0 += 32) {
            float incl = i0 + lane < n_list ? L.e[i0 + lane] : 0.f;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
              const float up = __shfl_up_sync(0xffffffffu, incl, o);
              if (lane >= o) incl += up;
            }
            if (i0 + lane < n_list) L.e[i0 + lane] = run + incl;
            run += __shfl_sync(0xffffffffu, incl, 31);
          }
          __syncwarp();
          // first place among the first m whose cumulative sum reaches target (m if none does)
          auto reaching = [&](float target, int m) {
            int lo = 0, hi = m;
            while (lo < hi) {
              const int mid = (lo + hi) >> 1;
              if (L.e[mid] >= target) hi = mid; else lo = mid + 1;
            }
            return lo;
          };
          int n_keep = n_list;
          if (top_p < 1.f) {
            // shortest head (descending) whose cumulative probability reaches top_p
            const int j = reaching(top_p * L.e[n_list - 1], n_list);
            if (j < n_list) n_keep = j + 1;
          }
          const int j = reaching(u * L.e[n_keep - 1], n_keep);
          if (lane == 0) {
            keep(L.idx[j < n_keep ? j : n_keep - 1]);
            s_done = 1;
          }
        }
      } else if (threadIdx.x == 0) {
        int n_keep = n_list;
        bool done = true;
        float kept = 0.f;
        if (cut_k) for (int j = 0; j < n_keep; ++j) kept += L.e[j];
        else kept = whole;
        if (top_p < 1.f) {
          // shortest head (descending) whose cumulative probability reaches top_p
          const float target = top_p * kept;
          float run = 0.f;
          done = cut_k;                             // a top_k's list always holds the head; the best 512 may not
          for (int j = 0; j < n_keep; ++j) {
            run += L.e[j];
            if (run >= target) { n_keep = j + 1; done = true; break; }
          }
          kept = 0.f;
          for (int j = 0; j < n_keep; ++j) kept += L.e[j];
        }
        s_done = done ? 1 : 0;
        if (done) {
          const float target = u * kept;
          float run = 0.f;
          int pick = L.idx[n_keep - 1];
          for (int j = 0; j < n_keep; ++j) {
            run += L.e[j];
            if (run >= target) { pick = L.idx[j]; break; }
          }
          keep(pick);
        }
      }
      __syncthreads();
      G2B_STAMP(11);
      if (s_done) return;
    }
    __syncthreads();
  }
  block_argmax(row, V, inv_temp, &mx);

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
  draw();
  const float target = u * kept;
  const Descent d = radix_descent<true>(row, V, inv_temp, mx, bound_key, bounded, target, hist);
  int choice = tie_walk<true>(row, V, inv_temp, mx, d.key, d.above, target, tie_list);
  if (bounded && d.key == bound_key && choice > tie_idx) choice = tie_idx;
  if (threadIdx.x == 0) keep(choice < 0 ? 0 : choice);
}

// recent: [R, recent_ld] ids, recent_n[R] how many are valid; or recent == nullptr: the last
// ids of every row's sequence are in its record (seq_state[slots[row]]), and with `append` the
// chosen id is added to them.  logits are modified in place by the penalty.  cand: scratch of
// g2b_sample_filtered_scratch_words(R) ints, or null; with it, a small top_k over a large
// vocabulary is listed by many blocks per row first (filter_slices_kernel).
static int g2b_sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

extern "C" int g2b_sample_filtered_scratch_words(int R) {
  return (int)min((long long)R * ROW_CAND_WORDS, (long long)INT_MAX);
}

extern "C" int g2b_sample_filtered(float *logits, int R, int V, int ld, float temp, int top_k,
                                   float top_p, float penalty, const int *recent, int recent_ld,
                                   const int *recent_n, int *seq_state, int state_words,
                                   const int *slots, int *out_ids, int append, int *cand,
                                   cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0 || ld < V) G2B_REFUSE("sample_filtered: bad sizes V=%d ld=%d", V, ld);
  if (!(top_p > 0.f)) G2B_REFUSE("sample_filtered: top_p must be in (0, 1], got %g", top_p);
  if (!(penalty > 0.f)) G2B_REFUSE("sample_filtered: repeat penalty must be positive, got %g", penalty);
  if (temp > 0.f && (!seq_state || !slots || state_words < 4))
    G2B_REFUSE("sample_filtered: temperature sampling needs the per-slot state");
  if (!recent && penalty != 1.f && (!seq_state || !slots || state_words < SS_RING + SS_RING_WORDS))
    G2B_REFUSE("sample_filtered: a repeat penalty without the recent ids needs the per-slot records with their rings");
  // slices per row: as many as there are lists while that is at most about one round of blocks (three of
  // them fit an SM), else half as many, down to 4
  int n_slices = 2048 / slice_cap(top_k);
  while (n_slices > 4 && (long long)n_slices * R > 3LL * g2b_sm_count()) n_slices >>= 1;
  const bool slices = cand && temp > 0.f && top_k > 0 && top_k <= MAX_SLICE_CAP && V >= 8192 &&
                      (long long)n_slices * R <= 3LL * g2b_sm_count();
  if (slices) {
    g2b_launch(filter_slices_kernel, dim3(n_slices, R), dim3(FILTER_THREADS), 0, stream,
        logits, V, ld, temp, top_k, penalty, recent, recent_ld, recent_n, (const int *)seq_state, state_words,
        slots, cand);
    int rc = g2b_check_launch("sample_filtered (slices)");
    if (rc) return rc;
  }
  g2b_launch(sample_filtered_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream,
      logits, V, ld, temp, top_k, top_p, penalty, recent, recent_ld, recent_n, seq_state,
      state_words, slots, out_ids, append, (const int *)(slices ? cand : nullptr));
  return g2b_check_launch("sample_filtered");
}

// Starts the rings of recent ids of the given slots: src [n, 1 + RECENT_WINDOW] = count, ids
// (oldest first).
__global__ void recent_set_kernel(int *seq_state, int words, const int *slots, const int *src, int n) {
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  if (r >= n) return;
  int *rec = seq_state + (size_t)slots[r] * words;
  const int *row = src + (size_t)r * (1 + RECENT_WINDOW);
  const int count = min(max(row[0], 0), RECENT_WINDOW);
  for (int i = threadIdx.x; i < count; i += blockDim.x) rec[SS_RING + i] = row[1 + i];
  if (threadIdx.x == 0) rec[SS_RECENT_TOTAL] = count;
}

extern "C" int g2b_recent_set(int *seq_state, int words, const int *slots, const int *src, int n,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  if (words < SS_RING + SS_RING_WORDS) G2B_REFUSE("recent_set: records of %d words have no ring", words);
  g2b_launch(recent_set_kernel, dim3(n), dim3(64), 0, stream, seq_state, words, slots, src, n);
  return g2b_check_launch("recent_set");
}

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
