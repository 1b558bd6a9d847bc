// Decode attention over the paged bfloat16 cache, split along the keys.
//
// One token per query row: every token t of the step attends, for each of its query
// heads, to the keys 0..pos_t of its own sequence (optionally only the last `window`).
// Grid (key chunk, kv head x head tile, token): a CTA takes one chunk of CHUNK_KEYS keys
// (chunks start at absolute positions that are multiples of CHUNK_KEYS, so the split of
// a token's keys depends on nothing but its position) and ALL query heads that share the
// kv head: they are the rows of a 16-row tensor-core tile, so K and V are read once per
// group.  Each warp streams whole pages: K and V panels of a (page, kv head) are
// contiguous, copied with 16-byte cp.async into XOR-swizzled shared memory and read back
// with ldmatrix; while a warp computes on K the V of the same page is in flight, while it
// computes P.V the next K is.  Scores, softmax statistics and the output are 32-bit;
// probabilities are rounded to bfloat16 for the P.V product.
//
// Each CTA writes an unnormalised partial output with its maximum and sum (log2 domain)
// to scratch; `attn_combine_kernel` merges a token's chunks in an order that depends on its
// position only.
//
// Formula: src/l5_model.c:518, 559-577 of AnonymoDGH/gguf2bin.  Compiled per head size
// (-DHD=64 or 128); the page size is 64 keys.
#include "common.cuh"
#include "mma.cuh"

G2B_DEFINE_LAST_ERROR

#ifndef HD
#define HD 128
#endif
static_assert(HD == 64 || HD == 128, "attn_decode: head sizes 64 and 128");

constexpr int PAGE = 64;                       // keys per page
constexpr int ROW_BYTES = HD * 2;
constexpr int ROW_CHUNKS = HD / 8;             // 16-byte pieces per row
constexpr int PANEL_BYTES = PAGE * ROW_BYTES;  // one (page, kv head) panel of K or of V
#ifndef ATTN_DECODE_WARPS
#define ATTN_DECODE_WARPS 2
#endif
#ifndef ATTN_DECODE_PAGES
#define ATTN_DECODE_PAGES 4
#endif
constexpr int WARPS = ATTN_DECODE_WARPS;
constexpr int PAGES_PER_CTA = ATTN_DECODE_PAGES;
constexpr int CHUNK_KEYS = PAGE * PAGES_PER_CTA;
constexpr int KSTEPS = HD / 16;                // k-steps of q.k over the head size
constexpr int DTILES = HD / 8;                 // n-tiles of the output over the head size
constexpr float LOG2E = 1.4426950408889634f;

// byte offset of (row, 16-byte piece) in a swizzled panel
__device__ __forceinline__ uint32_t swz(int row, int piece) {
  return (uint32_t)(row * ROW_BYTES + ((piece ^ (row & 7)) << 4));
}

// a load that is neither cached in registers across the dependency line nor merged with another
__device__ __forceinline__ int ld_volatile(const int *p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void load_panel(uint32_t smem_panel, const bf16 *gpanel, int lane) {
  // PAGE * ROW_CHUNKS pieces, 32 lanes
#pragma unroll
  for (int i = 0; i < PAGE * ROW_CHUNKS / 32; ++i) {
    const int idx = i * 32 + lane;
    const int row = idx / ROW_CHUNKS, piece = idx % ROW_CHUNKS;
    cp_async_16(smem_panel + swz(row, piece), gpanel + (size_t)row * HD + piece * 8);
  }
}

// What a warp accumulates over its pages: the unnormalised output of the tile's 16 query rows
// (lane (g, c) holds rows g and g + 8, columns 8n + 2c, 8n + 2c + 1), their running maxima
// (log2 domain) and sums.
struct Partial {
  float o[DTILES][4];
  float m[2], l[2];
};

// The query rows of a tile as A fragments: head = kvh * group + ht * 16 + row.
__device__ __forceinline__ void load_q_tile(uint32_t (&qa)[KSTEPS][4], const bf16 *__restrict__ q, int t,
                                            int nh, int kvh, int group, int ht, int g, int c) {
  const int row0 = ht * 16 + g, row1 = row0 + 8;
  const bf16 *q0 = q + ((size_t)t * nh + (size_t)kvh * group + row0) * HD;
  const bf16 *q1 = q0 + 8 * HD;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    const int d = ks * 16 + 2 * c;
    qa[ks][0] = row0 < group ? *reinterpret_cast<const uint32_t *>(q0 + d) : 0u;
    qa[ks][1] = row1 < group ? *reinterpret_cast<const uint32_t *>(q1 + d) : 0u;
    qa[ks][2] = row0 < group ? *reinterpret_cast<const uint32_t *>(q0 + d + 8) : 0u;
    qa[ks][3] = row1 < group ? *reinterpret_cast<const uint32_t *>(q1 + d + 8) : 0u;
  }
}

// One warp over the pages pg0, pg0 + stride, ... (n_pages of them, each holding a visible key):
// K and V panels through the warp's two buffers; while it computes on K the V of the same page
// is in flight, while it computes P.V the next K is.  The first K and V must have been issued
// (one commit group each) before the call.
template <typename PanelOf>
__device__ __forceinline__ void attend_pages(Partial &acc, const uint32_t (&qa)[KSTEPS][4], uint32_t k_smem,
                                             uint32_t v_smem, int pg0, int stride, int n_pages, int pos, int lo,
                                             float scale_log2, int lane, PanelOf panel_of) {
  const int g = lane >> 2, c = lane & 3;
  (void)g;
  float (&o)[DTILES][4] = acc.o;
  float (&m)[2] = acc.m, (&l)[2] = acc.l;
  for (int i = 0; i < n_pages; ++i) {
    const int key0 = (pg0 + i * stride) * PAGE;
    cp_async_wait<1>();                    // this page's K has landed (its V may be in flight)
    __syncwarp();
    float s[PAGE / 8][4];
#pragma unroll
    for (int j = 0; j < PAGE / 8; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int kp = 0; kp < KSTEPS / 2; ++kp) {
        uint32_t kb[4];
        ldmatrix_x4(kb, k_smem + swz(8 * j + (lane & 7), 4 * kp + (lane >> 3)));
        mma_bf16_16816(s[j], qa[2 * kp], kb[0], kb[1]);
        mma_bf16_16816(s[j], qa[2 * kp + 1], kb[2], kb[3]);
      }
    }
    __syncwarp();                          // every lane is done reading K
    if (i + 1 < n_pages) load_panel(k_smem, panel_of(pg0 + (i + 1) * stride, 0), lane);
    cp_async_commit();

    // scale (log2 domain), mask, running maximum and sum
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < PAGE / 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + 8 * j + 2 * c + (e & 1);
        const float v = (key <= pos && key >= lo) ? s[j][e] * scale_log2 : -INFINITY;
        s[j][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m[r], mx[r]);          // finite: the page holds a visible key
      corr[r] = fast_exp2(m[r] - m_new);
      m[r] = m_new;
      l[r] *= corr[r];
    }
    uint32_t pa[PAGE / 16][4];
#pragma unroll
    for (int j = 0; j < PAGE / 8; ++j) {
      const float p0 = fast_exp2(s[j][0] - m[0]), p1 = fast_exp2(s[j][1] - m[0]);
      const float p2 = fast_exp2(s[j][2] - m[1]), p3 = fast_exp2(s[j][3] - m[1]);
      l[0] += p0 + p1;
      l[1] += p2 + p3;
      pa[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
      pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int n = 0; n < DTILES; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0];
      o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }

    cp_async_wait<1>();                    // this page's V has landed (the next K may be in flight)
    __syncwarp();
#pragma unroll
    for (int kk = 0; kk < PAGE / 16; ++kk) {
#pragma unroll
      for (int dp = 0; dp < DTILES / 2; ++dp) {
        uint32_t vb[4];
        // matrices: (keys +0..7, d tile 2dp), (keys +8..15, d tile 2dp), (keys +0..7, 2dp+1), (+8..15, 2dp+1)
        const int mi = lane >> 3;
        ldmatrix_x4_trans(vb, v_smem + swz(16 * kk + (mi & 1) * 8 + (lane & 7), 2 * dp + (mi >> 1)));
        mma_bf16_16816(o[2 * dp], pa[kk], vb[0], vb[1]);
        mma_bf16_16816(o[2 * dp + 1], pa[kk], vb[2], vb[3]);
      }
    }
    __syncwarp();
    if (i + 1 < n_pages) load_panel(v_smem, panel_of(pg0 + (i + 1) * stride, 1), lane);
    cp_async_commit();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
}

// The warps of a CTA merged into warp 0, in warp order, through shared memory `xo`
// ([n_warps][32 lanes][DTILES * 4 + 4] floats; the panels are no longer needed).  Every thread
// of the CTA calls it.
__device__ __forceinline__ void merge_warps(Partial &acc, float *xo, int n_warps, int warp, int lane) {
  float (&o)[DTILES][4] = acc.o;
  float (&m)[2] = acc.m, (&l)[2] = acc.l;
  constexpr int PER_LANE = DTILES * 4 + 4;
  __syncthreads();
  if (warp > 0) {
    float *dst = xo + ((size_t)warp * 32 + lane) * PER_LANE;
#pragma unroll
    for (int n = 0; n < DTILES; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) dst[n * 4 + e] = o[n][e];
    dst[DTILES * 4 + 0] = m[0]; dst[DTILES * 4 + 1] = m[1];
    dst[DTILES * 4 + 2] = l[0]; dst[DTILES * 4 + 3] = l[1];
  }
  __syncthreads();
  if (warp == 0) {
    for (int w = 1; w < n_warps; ++w) {
      const float *src = xo + ((size_t)w * 32 + lane) * PER_LANE;
      float a[2], bb[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float mo = src[DTILES * 4 + r];
        const float m_new = fmaxf(m[r], mo);
        a[r] = m[r] == -INFINITY ? 0.f : fast_exp2(m[r] - m_new);
        bb[r] = mo == -INFINITY ? 0.f : fast_exp2(mo - m_new);
        l[r] = l[r] * a[r] + src[DTILES * 4 + 2 + r] * bb[r];
        m[r] = m_new;
      }
#pragma unroll
      for (int n = 0; n < DTILES; ++n) {
        o[n][0] = o[n][0] * a[0] + src[n * 4 + 0] * bb[0];
        o[n][1] = o[n][1] * a[0] + src[n * 4 + 1] * bb[0];
        o[n][2] = o[n][2] * a[1] + src[n * 4 + 2] * bb[1];
        o[n][3] = o[n][3] * a[1] + src[n * 4 + 3] * bb[1];
      }
    }
  }
}

__device__ __forceinline__ void clear_partial(Partial &acc) {
#pragma unroll
  for (int n = 0; n < DTILES; ++n) acc.o[n][0] = acc.o[n][1] = acc.o[n][2] = acc.o[n][3] = 0.f;
  acc.m[0] = acc.m[1] = -INFINITY;
  acc.l[0] = acc.l[1] = 0.f;
}

__global__ void __launch_bounds__(WARPS * 32)
attn_decode_kernel(const bf16 *__restrict__ q, const bf16 *__restrict__ cache,
                   const int *__restrict__ tok_pos, const int *__restrict__ tok_seq,
                   const int *__restrict__ page_table, int P, int nh, int nkv, int window,
                   float scale_log2, float *__restrict__ part_o, float2 *__restrict__ part_ml,
                   int n_chunks) {
  pdl_launch();
  extern __shared__ __align__(128) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int group = nh / nkv;
  const int head_tiles = (group + 15) / 16;
  const int chunk = blockIdx.x;
  const int kvh = blockIdx.y / head_tiles, ht = blockIdx.y % head_tiles;
  const int t = blockIdx.z;
  const int key_begin = chunk * CHUNK_KEYS;
  const int first_page = key_begin / PAGE;
  unsigned char *my = smem + warp * 2 * PANEL_BYTES;
  const uint32_t k_smem = smem_u32(my), v_smem = smem_u32(my + PANEL_BYTES);
  const size_t panel_elems = (size_t)PAGE * HD;
  // the batch's layout (which sequence, which pages) was copied to the device before the step's
  // first kernel was launched, so it may be read above the dependency line
  const int b = tok_seq[t];
  auto panel_of = [&](int pg, int kv) {
    const int phys = page_table[(size_t)b * P + pg];
    return cache + (((size_t)phys * 2 + kv) * nkv + kvh) * panel_elems;
  };

  // Before the kernels in front of this one are done (they compute this token's query and
  // write its key and value), the warp's first page can already be on its way if it is an OLD
  // page: one that lies wholly below the token's position and was therefore completed by an
  // earlier step.  The position itself is moved on the device by earlier kernels (one forward
  // at the end of every step; one back when a step that was launched ahead is taken back), so
  // what is read here is a hint: it may lag behind by any number of steps, which is harmless
  // (whichever value is seen was written after every key below it), and it may be one too
  // large while a take-back is still on its way, which the "- 1" allows for.  Not with a
  // window, whose lower edge moves with the position.
  const int hint = ld_volatile(tok_pos + t);
  const bool early = window <= 0 && (first_page + warp + 1) * PAGE <= hint - 1;
  if (early) {
    load_panel(k_smem, panel_of(first_page + warp, 0), lane);
    cp_async_commit();
    load_panel(v_smem, panel_of(first_page + warp, 1), lane);
    cp_async_commit();
  }
  pdl_wait();
  const int pos = ld_volatile(tok_pos + t);
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  if (key_begin > pos || key_begin + CHUNK_KEYS <= lo) return;     // no key of this chunk is seen (then nothing was fetched early)

  // the pages of this warp: key_begin/PAGE + warp, + WARPS, ... that hold a visible key (the
  // visible pages of a chunk are a contiguous range)
  int pg0 = 0, n_pages = 0;
#pragma unroll
  for (int i = 0; i < PAGES_PER_CTA / WARPS; ++i) {
    const int pg = first_page + warp + i * WARPS;
    if (pg * PAGE <= pos && (pg + 1) * PAGE > lo) {
      if (n_pages == 0) pg0 = pg;
      ++n_pages;
    }
  }
  if (!early) {
    if (n_pages > 0) load_panel(k_smem, panel_of(pg0, 0), lane);
    cp_async_commit();
    if (n_pages > 0) load_panel(v_smem, panel_of(pg0, 1), lane);
    cp_async_commit();
  }

  uint32_t qa[KSTEPS][4];
  load_q_tile(qa, q, t, nh, kvh, group, ht, g, c);
  Partial acc;
  clear_partial(acc);
  attend_pages(acc, qa, k_smem, v_smem, pg0, WARPS, n_pages, pos, lo, scale_log2, lane, panel_of);
  merge_warps(acc, reinterpret_cast<float *>(smem), WARPS, warp, lane);
  if (warp == 0) {
    float (&o)[DTILES][4] = acc.o;
    float (&m)[2] = acc.m, (&l)[2] = acc.l;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = ht * 16 + g + 8 * r;
      if (row >= group) continue;
      const size_t slot = ((size_t)t * nh + (size_t)kvh * group + row) * n_chunks + chunk;
      float *po = part_o + slot * HD;
#pragma unroll
      for (int n = 0; n < DTILES; ++n)
        *reinterpret_cast<float2 *>(po + 8 * n + 2 * c) = make_float2(o[n][2 * r], o[n][2 * r + 1]);
      if (c == 0) part_ml[slot] = make_float2(m[r], l[r]);
    }
  }
}

// out[t, h, :] = sum_i 2^(m_i - M) o_i / sum_i 2^(m_i - M) l_i over the token's chunks.  One block of
// four warps per (token, head): warp w adds the chunks c0 + w, c0 + w + 4, ... in that order, a lane
// four neighbouring elements of the head; the four sums are then added in the order of the warps.
// The order depends on the token's position only.
constexpr int COMBINE_WARPS = 4;
__global__ void __launch_bounds__(COMBINE_WARPS * 32)
attn_combine_kernel(const float *__restrict__ part_o, const float2 *__restrict__ part_ml,
                    const int *__restrict__ tok_pos, int nh, int window, int n_chunks,
                    bf16 *__restrict__ out) {
  pdl_launch();
  pdl_wait();
  __shared__ float s_max[COMBINE_WARPS];
  __shared__ float s_acc[COMBINE_WARPS][HD + 1];
  const size_t th = blockIdx.x;                                // t * nh + h
  const int t = (int)(th / nh);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = tok_pos[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int c0 = lo / CHUNK_KEYS, c1 = pos / CHUNK_KEYS;
  const float2 *ml = part_ml + th * n_chunks;
  float M = -INFINITY;
  for (int i = c0 + (int)threadIdx.x; i <= c1; i += COMBINE_WARPS * 32) M = fmaxf(M, ml[i].x);
  M = warp_max(M);
  if (lane == 0) s_max[warp] = M;
  __syncthreads();
  M = fmaxf(fmaxf(s_max[0], s_max[1]), fmaxf(s_max[2], s_max[3]));
  const bool active = 4 * lane < HD;
  float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
  float den = 0.f;
  // eight chunks' loads in flight at a time (a token far into its sequence has hundreds of chunks,
  // and one load after the other cost 20 us at 65,536 keys); they are added in the same order
  constexpr int AHEAD = 8;
  for (int i0 = c0 + warp; i0 <= c1; i0 += AHEAD * COMBINE_WARPS) {
    float2 mlv[AHEAD];
    float4 ov[AHEAD];
#pragma unroll
    for (int u = 0; u < AHEAD; ++u) {
      const int i = i0 + u * COMBINE_WARPS;
      if (i <= c1) {
        mlv[u] = ml[i];
        if (active) ov[u] = *reinterpret_cast<const float4 *>(part_o + (th * n_chunks + i) * HD + 4 * lane);
      }
    }
#pragma unroll
    for (int u = 0; u < AHEAD; ++u) {
      if (i0 + u * COMBINE_WARPS <= c1) {
        const float w = fast_exp2(mlv[u].x - M);
        if (active) {
          num.x = fmaf(w, ov[u].x, num.x); num.y = fmaf(w, ov[u].y, num.y);
          num.z = fmaf(w, ov[u].z, num.z); num.w = fmaf(w, ov[u].w, num.w);
        }
        den = fmaf(w, mlv[u].y, den);
      }
    }
  }
  if (active) {
    s_acc[warp][4 * lane] = num.x; s_acc[warp][4 * lane + 1] = num.y;
    s_acc[warp][4 * lane + 2] = num.z; s_acc[warp][4 * lane + 3] = num.w;
  }
  if (lane == 0) s_acc[warp][HD] = den;
  __syncthreads();
  for (int d = threadIdx.x; d < HD; d += COMBINE_WARPS * 32) {
    const float n = ((s_acc[0][d] + s_acc[1][d]) + s_acc[2][d]) + s_acc[3][d];
    const float dn = ((s_acc[0][HD] + s_acc[1][HD]) + s_acc[2][HD]) + s_acc[3][HD];
    out[th * HD + d] = __float2bfloat16_rn(n / dn);
  }
}

// Scratch: part_o float [T*nh*n_chunks*HD], part_ml float2 [T*nh*n_chunks], with
// n_chunks = ceil(max_kv_len / 256).  q, out [T, nh*HD] bfloat16.
// With programmatic dependent launch on (g2b_set_pdl(1)) the kernel reads tok_pos once above
// the dependency line, as a hint for which old pages it may fetch early.  A caller whose own
// kernels move tok_pos while this one may already have started must keep to what the library
// does: positions grow, and shrink by at most one (a step taken back) between two launches.
// With ordinary launches (the default of a freshly loaded object) there is no such rule.
extern "C" int g2b_attn_decode(const void *q, void *out, const void *cache, const int *tok_pos,
                               const int *tok_seq, const int *page_table, int P, int T, int nh,
                               int nkv, int hd, int page_size, int window, float scale,
                               int max_kv_len, float *part_o, float *part_ml,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd != HD) G2B_REFUSE("attn_decode: built for head_dim %d, got %d", HD, hd);
  if (page_size != PAGE) G2B_REFUSE("attn_decode: page size must be %d, got %d", PAGE, page_size);
  if (nkv <= 0 || nh % nkv) G2B_REFUSE("attn_decode: %d heads are not a multiple of %d kv heads", nh, nkv);
  if (T > 65535) G2B_REFUSE("attn_decode: %d tokens in one step (at most 65535)", T);
  const int group = nh / nkv, head_tiles = (group + 15) / 16;
  if ((long long)nkv * head_tiles > 65535) G2B_REFUSE("attn_decode: too many kv heads (%d)", nkv);
  const int n_chunks = (max_kv_len + CHUNK_KEYS - 1) / CHUNK_KEYS;
  if (n_chunks <= 0) G2B_REFUSE("attn_decode: max_kv_len %d", max_kv_len);
  const int smem = WARPS * 2 * PANEL_BYTES;
  static G2bPerDevice configured;
  const int cfg_dev = g2b_current_device();
  if (cfg_dev < 0 || !configured.value[cfg_dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) G2B_REFUSE("attn_decode: shared memory of %d bytes refused: %s", smem, cudaGetErrorString(e));
    if (cfg_dev >= 0) configured.value[cfg_dev] = 1;
  }
  dim3 grid(n_chunks, nkv * head_tiles, T);
  g2b_launch(attn_decode_kernel, dim3(grid), dim3(WARPS * 32), smem, stream, 
      (const bf16 *)q, (const bf16 *)cache, tok_pos, tok_seq, page_table, P, nh, nkv, window,
      scale * LOG2E, part_o, (float2 *)part_ml, n_chunks);
  int rc = g2b_check_launch("attn_decode");
  if (rc) return rc;
  g2b_launch(attn_combine_kernel, dim3((unsigned)((size_t)T * nh)), dim3(COMBINE_WARPS * 32), 0, stream, 
      part_o, (const float2 *)part_ml, tok_pos, nh, window, n_chunks, (bf16 *)out);
  return g2b_check_launch("attn_combine");
}

extern "C" int g2b_attn_decode_chunk_keys() { return CHUNK_KEYS; }
