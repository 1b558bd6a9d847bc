// Prompt attention over the paged bfloat16 cache: causal, grouped-query, ragged, with a
// past.  The keys and values of the step's own tokens are already in the cache when this
// runs (the fused norm + rotation kernel wrote them), so past and present keys are read
// the same way, page by page.
//
// Work list: the host cuts every sequence's new tokens into tiles of 64 query rows and
// sends (sequence, first token index, rows, position of the first row) per tile, longest
// first.  Grid (tile, query head).  A CTA of 4 warps holds 16 query rows per warp as
// tensor-core A fragments and walks the key pages 0 .. page of its last row (or from the
// window's first page): the K and V panels of a (page, kv head) are contiguous 16 KB
// (head size 128), copied by all threads with 16-byte cp.async into XOR-swizzled shared
// memory, double-buffered, read with ldmatrix.  Scores, running maximum and sum, and the
// output accumulate in 32-bit; probabilities are rounded to bfloat16 for P.V.  Masks
// (causal, window) are applied only on pages that cross a row's limits.  A row's key
// tiles are the pages, whatever the step's shape: its arithmetic depends only on its own
// position.
//
// Formula: src/l5_model.c:518, 559-577 of AnonymoDGH/gguf2bin.  Compiled per head size
// (-DHD=64 or 128); pages hold 64 keys.
#include "common.cuh"
#include "mma.cuh"

G2B_DEFINE_LAST_ERROR

#ifndef HD
#define HD 128
#endif
static_assert(HD == 64 || HD == 128, "attn_prefill: head sizes 64 and 128");

constexpr int PAGE = 64;
constexpr int ROW_BYTES = HD * 2;
constexpr int ROW_CHUNKS = HD / 8;
constexpr int PANEL_BYTES = PAGE * ROW_BYTES;
constexpr int WARPS = 4;
constexpr int BM = WARPS * 16;                 // query rows per tile
constexpr int KSTEPS = HD / 16;
constexpr int DTILES = HD / 8;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t swz(int row, int piece) {
  return (uint32_t)(row * ROW_BYTES + ((piece ^ (row & 7)) << 4));
}

__device__ __forceinline__ void load_panel(uint32_t smem_panel, const bf16 *gpanel, int tid) {
#pragma unroll
  for (int i = 0; i < PAGE * ROW_CHUNKS / (WARPS * 32); ++i) {
    const int idx = i * (WARPS * 32) + tid;
    const int row = idx / ROW_CHUNKS, piece = idx % ROW_CHUNKS;
    cp_async_16(smem_panel + swz(row, piece), gpanel + (size_t)row * HD + piece * 8);
  }
}

// tiles: [n_tiles][4] = {sequence index, first token index, rows, position of row 0}
__global__ void __launch_bounds__(WARPS * 32, 3)
attn_prefill_kernel(const bf16 *__restrict__ q, bf16 *__restrict__ out,
                    const bf16 *__restrict__ cache, const int4 *__restrict__ tiles,
                    const int *__restrict__ page_table, int P, int nh, int nkv, int window,
                    float scale_log2) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int4 tile = tiles[blockIdx.x];
  const int b = tile.x, t0 = tile.y, n_rows = tile.z, pos0 = tile.w;
  const int h = blockIdx.y, kvh = h / (nh / nkv);

  const int last_pos = pos0 + n_rows - 1;
  const int first_page = window > 0 ? max(0, pos0 - window + 1) / PAGE : 0;
  const int last_page = last_pos / PAGE;

  const size_t panel_elems = (size_t)PAGE * HD;
  const int *pt = page_table + (size_t)b * P;
  auto issue_page = [&](int pg, int stage) {
    const int phys = pt[pg];
    const bf16 *kp = cache + (((size_t)phys * 2 + 0) * nkv + kvh) * panel_elems;
    const bf16 *vp = cache + (((size_t)phys * 2 + 1) * nkv + kvh) * panel_elems;
    const uint32_t base = smem_u32(smem) + stage * 2 * PANEL_BYTES;
    load_panel(base, kp, tid);
    load_panel(base + PANEL_BYTES, vp, tid);
  };
  issue_page(first_page, 0);
  cp_async_commit();

  // this warp's 16 query rows as A fragments (rows past the tile's end are zero)
  const int r0 = warp * 16 + g, r1 = r0 + 8;
  const bf16 *q0 = q + ((size_t)(t0 + r0) * nh + h) * HD;
  const bf16 *q1 = q + ((size_t)(t0 + r1) * nh + h) * HD;
  uint32_t qa[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    const int d = ks * 16 + 2 * c;
    qa[ks][0] = r0 < n_rows ? *reinterpret_cast<const uint32_t *>(q0 + d) : 0u;
    qa[ks][1] = r1 < n_rows ? *reinterpret_cast<const uint32_t *>(q1 + d) : 0u;
    qa[ks][2] = r0 < n_rows ? *reinterpret_cast<const uint32_t *>(q0 + d + 8) : 0u;
    qa[ks][3] = r1 < n_rows ? *reinterpret_cast<const uint32_t *>(q1 + d + 8) : 0u;
  }
  const int pos_r[2] = {pos0 + r0, pos0 + r1};
  const int lo_r[2] = {window > 0 ? max(0, pos_r[0] - window + 1) : 0,
                       window > 0 ? max(0, pos_r[1] - window + 1) : 0};
  const int warp_pos_min = pos0 + warp * 16, warp_pos_max = warp_pos_min + 15;
  const int warp_lo_max = window > 0 ? max(0, warp_pos_max - window + 1) : 0;
  const int warp_lo_min = window > 0 ? max(0, warp_pos_min - window + 1) : 0;

  float o[DTILES][4];
#pragma unroll
  for (int n = 0; n < DTILES; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  for (int pg = first_page; pg <= last_page; ++pg) {
    const int stage = (pg - first_page) & 1;
    if (pg + 1 <= last_page) issue_page(pg + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int key0 = pg * PAGE;
    // pages wholly after this warp's rows, or wholly before their windows, are skipped
    const bool seen = key0 <= warp_pos_max && key0 + PAGE > warp_lo_min;
    if (seen) {
      const uint32_t k_smem = smem_u32(smem) + stage * 2 * PANEL_BYTES;
      const uint32_t v_smem = k_smem + PANEL_BYTES;
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
      const bool partial = key0 + PAGE - 1 > warp_pos_min || key0 < warp_lo_max;
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < PAGE / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[j][e] * scale_log2;
          if (partial) {
            const int key = key0 + 8 * j + 2 * c + (e & 1);
            if (key > pos_r[e >> 1] || key < lo_r[e >> 1]) v = -INFINITY;
          }
          s[j][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      float corr[2], msafe[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m[r], mx[r]);
        msafe[r] = m_new == -INFINITY ? 0.f : m_new;      // a row that has seen no key yet
        corr[r] = fast_exp2(m[r] - msafe[r]);
        m[r] = m_new;
        l[r] *= corr[r];
      }
      uint32_t pa[PAGE / 16][4];
#pragma unroll
      for (int j = 0; j < PAGE / 8; ++j) {
        const float p0 = fast_exp2(s[j][0] - msafe[0]), p1 = fast_exp2(s[j][1] - msafe[0]);
        const float p2 = fast_exp2(s[j][2] - msafe[1]), p3 = fast_exp2(s[j][3] - msafe[1]);
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
#pragma unroll
      for (int kk = 0; kk < PAGE / 16; ++kk) {
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) {
          uint32_t vb[4];
          const int mi = lane >> 3;
          ldmatrix_x4_trans(vb, v_smem + swz(16 * kk + (mi & 1) * 8 + (lane & 7), 2 * dp + (mi >> 1)));
          mma_bf16_16816(o[2 * dp], pa[kk], vb[0], vb[1]);
          mma_bf16_16816(o[2 * dp + 1], pa[kk], vb[2], vb[3]);
        }
      }
    }
    __syncthreads();                       // this stage is overwritten by the copy after next
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    const int row = warp * 16 + g + 8 * r;
    if (row >= n_rows) continue;
    const float inv = 1.f / l[r];
    bf16 *op = out + ((size_t)(t0 + row) * nh + h) * HD;
#pragma unroll
    for (int n = 0; n < DTILES; ++n)
      *reinterpret_cast<uint32_t *>(op + 8 * n + 2 * c) = pack_bf16(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
  }
}

extern "C" int g2b_attn_prefill(const void *q, void *out, const void *cache, const int *tiles,
                                int n_tiles, const int *page_table, int P, int nh, int nkv, int hd,
                                int page_size, int window, float scale, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (hd != HD) G2B_REFUSE("attn_prefill: built for head_dim %d, got %d", HD, hd);
  if (page_size != PAGE) G2B_REFUSE("attn_prefill: page size must be %d, got %d", PAGE, page_size);
  if (nkv <= 0 || nh % nkv) G2B_REFUSE("attn_prefill: %d heads are not a multiple of %d kv heads", nh, nkv);
  if (nh > 65535) G2B_REFUSE("attn_prefill: %d heads", nh);
  const int smem = 2 * 2 * PANEL_BYTES;
  static G2bPerDevice configured;
  const int cfg_dev = g2b_current_device();
  if (cfg_dev < 0 || !configured.value[cfg_dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) G2B_REFUSE("attn_prefill: shared memory of %d bytes refused: %s", smem, cudaGetErrorString(e));
    if (cfg_dev >= 0) configured.value[cfg_dev] = 1;
  }
  dim3 grid(n_tiles, nh);
  g2b_launch(attn_prefill_kernel, dim3(grid), dim3(WARPS * 32), smem, stream, 
      (const bf16 *)q, (bf16 *)out, (const bf16 *)cache, (const int4 *)tiles, page_table, P, nh,
      nkv, window, scale * LOG2E);
  return g2b_check_launch("attn_prefill");
}

extern "C" int g2b_attn_prefill_tile_rows() { return BM; }
