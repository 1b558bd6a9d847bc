// Prompt attention on the 5th-generation tensor cores: causal, grouped-query, ragged, with
// a past, over the paged bfloat16 cache (the step's own keys are already in it).
//
// Work list: tiles of 128 query rows (sequence, first token index, rows, position of the
// first row), longest first; one CTA per (tile, query head), numbered tile-major so that the
// long tiles of every head start first and the short ones fill in behind them.  Two CTAs fit
// on an SM (shared memory and tensor memory are sized for that): while one waits on its
// softmax the other's products run.  Roles by warp:
//   warp 4, one thread  TMA producer: the 128 x HD query tile once, then per key page the K
//                       and V panels of (page, kv head), each as 64-column boxes with 128-byte
//                       swizzle, into a ring of three K panels and a ring of two V panels (K is
//                       free again as soon as its S product is done, V only after P.V).
//   warp 5, one thread  MMA issuer (tcgen05.mma, cta_group::1, kind::f16):
//                         S[128 x 64]  = Q K^T      (both operands K-major)  -> tensor memory,
//                                                    two S buffers, always one page ahead
//                         O[128 x HD] += P V        (P read from tensor memory, V read as
//                                                    an MN-major operand: keys are its K index)
//   warps 0..3          softmax, one thread per query row: reads its row of S with tcgen05.ld,
//                       scales (log2 domain), masks (causal, window), keeps a reference maximum
//                       and a sum in float, and writes P = 2^(s - m) as packed bfloat16 back
//                       into the first columns of the same S buffer (tcgen05.st), where the
//                       second product reads it.  O is rescaled in tensor memory only when a
//                       row's maximum has grown by more than 2^8 since its reference (the
//                       result is the same function of the scores; the factor just stays
//                       bounded), and is normalised and stored at the end.
// Issue order of the MMAs: S0, S1, [P0 ready] PV0, S2, [P1 ready] PV1, S3, ...: while the
// softmax warps work on page i, S of page i+1 is already there and P.V of page i-1 runs.
//
// Every mbarrier wait is bounded; a wait that gives up records a code in `*status`, all roles
// fall through to the common exit and the tensor memory is freed.
//
// Formula: src/l5_model.c:518, 559-577 of AnonymoDGH/gguf2bin.  -DHD=64 or 128; 64-key pages.
#include "common.cuh"
#include "tc_common.cuh"

G2B_DEFINE_LAST_ERROR

#ifndef HD
#define HD 128
#endif
static_assert(HD == 64 || HD == 128, "attn_prefill_tc: head sizes 64 and 128");

using namespace tc;

constexpr int PAGE = 64;
constexpr int BM = 128;
constexpr int THREADS = 192;
constexpr int K_STAGES = 3, V_STAGES = 2;
constexpr int SUBS = HD / 64;                       // 64-column boxes along the head dimension
constexpr int Q_SUB_BYTES = BM * 128;               // one 128 x 64 box
constexpr int Q_BYTES = SUBS * Q_SUB_BYTES;
constexpr int KV_SUB_BYTES = PAGE * 128;            // one 64 x 64 box
constexpr int KV_BYTES = SUBS * KV_SUB_BYTES;       // K (or V) of one page and kv head
constexpr int K_OFFSET = Q_BYTES, V_OFFSET = K_OFFSET + K_STAGES * KV_BYTES;
constexpr int BAR_OFFSET = V_OFFSET + V_STAGES * KV_BYTES;
constexpr int SMEM_TOTAL = BAR_OFFSET + 256;
// two CTAs per SM: 2 x (dynamic + 1 KB reserved) must stay within the 227 KB of an SM
static_assert(2 * (SMEM_TOTAL + 1024) <= 227 * 1024, "two CTAs per SM");
constexpr int O_COL0 = 128;                         // S buffers at columns 0..63 and 64..127, O from 128
constexpr int TMEM_COLS = 256;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.f;                 // log2 of the growth that triggers a rescale

enum { ST_PRODUCER = 11, ST_MMA = 12, ST_SOFTMAX = 13, ST_ALIGN = 14 };
static_assert(HD <= 128, "O uses columns 128..255");

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

__global__ void __launch_bounds__(THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_kv, bf16 *__restrict__ out,
                       const int4 *__restrict__ tiles, const int *__restrict__ page_table, int P,
                       int nh, int nkv, int window, float scale_log2, int *__restrict__ status) {
  pdl_launch();
  // The swizzled panels need 1024-byte alignment.  The kernel has no static shared memory, so
  // the dynamic part starts at the aligned base of the window; checked rather than assumed.
  extern __shared__ __align__(1024) unsigned char smem[];
  if (smem_addr(smem) & 1023u) {
    if (threadIdx.x == 0) atomicExch(status, ST_ALIGN);
    return;
  }
  unsigned char *q_smem = smem;
  unsigned char *k_smem = smem + K_OFFSET, *v_smem = smem + V_OFFSET;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + BAR_OFFSET);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 20);
  const uint32_t q_full = smem_addr(bars + 0);
  const uint32_t k_full0 = smem_addr(bars + 1), k_empty0 = smem_addr(bars + 4);       // [K_STAGES] each
  const uint32_t v_full0 = smem_addr(bars + 7), v_empty0 = smem_addr(bars + 9);       // [V_STAGES] each
  const uint32_t s_ready0 = smem_addr(bars + 11), p_ready0 = smem_addr(bars + 13);    // [2] each
  const uint32_t pv_done = smem_addr(bars + 15), o_ready = smem_addr(bars + 16);
  static_assert(K_STAGES == 3 && V_STAGES == 2, "barrier slots");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < K_STAGES; ++s) {
      mbar_init(k_full0 + 8 * s, 1);
      mbar_init(k_empty0 + 8 * s, 1);
    }
    for (int s = 0; s < V_STAGES; ++s) {
      mbar_init(v_full0 + 8 * s, 1);
      mbar_init(v_empty0 + 8 * s, 1);
    }
    for (int j = 0; j < 2; ++j) {
      mbar_init(s_ready0 + 8 * j, 1);
      mbar_init(p_ready0 + 8 * j, BM);
    }
    mbar_init(pv_done, 1);
    mbar_init(o_ready, 1);
    mbar_init_fence();
  }
  if (warp == 5) tmem_alloc(smem_addr(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();                                   // the queries and the cache come from earlier kernels

  const int4 tile = tiles[blockIdx.x / nh];
  const int b = tile.x, t0 = tile.y, n_rows = tile.z, pos0 = tile.w;
  const int h = blockIdx.x % nh, kvh = h / (nh / nkv);
  const int first_page = window > 0 ? max(0, pos0 - window + 1) / PAGE : 0;
  const int last_page = (pos0 + n_rows - 1) / PAGE;
  const int n_pages = last_page - first_page + 1;

  if (warp == 4) {
    if (lane == 0) {
      mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int sub = 0; sub < SUBS; ++sub)
        tma_load_2d(smem_addr(q_smem + sub * Q_SUB_BYTES), &map_q, h * HD + 64 * sub, t0, q_full);
      const int *pt = page_table + (size_t)b * P + first_page;
      auto load_k = [&](int i) -> bool {
        const int s = i % K_STAGES;
        if (i >= K_STAGES && !mbar_wait(k_empty0 + 8 * s, ((i / K_STAGES) - 1) & 1)) return false;
        const int row = ((pt[i] * 2 + 0) * nkv + kvh) * PAGE;
        const uint32_t dst = smem_addr(k_smem + s * KV_BYTES);
        mbar_expect_tx(k_full0 + 8 * s, KV_BYTES);
#pragma unroll
        for (int sub = 0; sub < SUBS; ++sub)
          tma_load_2d(dst + sub * KV_SUB_BYTES, &map_kv, 64 * sub, row, k_full0 + 8 * s);
        return true;
      };
      auto load_v = [&](int i) -> bool {
        const int s = i % V_STAGES;
        if (i >= V_STAGES && !mbar_wait(v_empty0 + 8 * s, ((i / V_STAGES) - 1) & 1)) return false;
        const int row = ((pt[i] * 2 + 1) * nkv + kvh) * PAGE;
        const uint32_t dst = smem_addr(v_smem + s * KV_BYTES);
        mbar_expect_tx(v_full0 + 8 * s, KV_BYTES);
#pragma unroll
        for (int sub = 0; sub < SUBS; ++sub)
          tma_load_2d(dst + sub * KV_SUB_BYTES, &map_kv, 64 * sub, row, v_full0 + 8 * s);
        return true;
      };
      // in the order of use: K0, K1, V0, K2, V1, K3, ...
      bool ok = load_k(0);
      for (int i = 0; i < n_pages && ok; ++i) {
        if (i + 1 < n_pages) ok = load_k(i + 1);
        if (ok) ok = load_v(i);
      }
      if (!ok) atomicExch(status, ST_PRODUCER);
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = instr_desc(BM, PAGE, false);
      constexpr uint32_t idesc_pv = instr_desc(BM, HD, true);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) atomicExch(status, ST_MMA);
      // S of page i into S buffer i % 2 (needs K of stage i % K_STAGES)
      auto issue_s = [&](int i) -> bool {
        const int s = i % K_STAGES;
        if (!mbar_wait(k_full0 + 8 * s, (i / K_STAGES) & 1)) { atomicExch(status, ST_MMA); return false; }
        tc_fence_after();
        const uint32_t k_addr = smem_addr(k_smem + s * KV_BYTES);
#pragma unroll
        for (int sub = 0; sub < SUBS; ++sub)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem + 64 * (i & 1), desc_k_major(smem_addr(q_smem + sub * Q_SUB_BYTES)) + 2 * k,
                      desc_k_major(k_addr + sub * KV_SUB_BYTES) + 2 * k, idesc_s, (sub | k) != 0);
        umma_commit(k_empty0 + 8 * s);             // K of this stage has been read
        umma_commit(s_ready0 + 8 * (i & 1));
        return true;
      };
      if (ok) ok = issue_s(0);
      if (ok && n_pages > 1) ok = issue_s(1);
      for (int i = 0; i < n_pages && ok; ++i) {
        const int s = i % V_STAGES;
        if (!mbar_wait(v_full0 + 8 * s, (i / V_STAGES) & 1) ||
            !mbar_wait(p_ready0 + 8 * (i & 1), (i >> 1) & 1)) { atomicExch(status, ST_MMA); break; }
        tc_fence_after();
        // O += P V: the keys are the K index, 16 per MMA: 8 packed columns of P, 16 rows of V
        const uint32_t v_addr = smem_addr(v_smem + s * KV_BYTES);
#pragma unroll
        for (int k = 0; k < PAGE / 16; ++k)
          umma_bf16_ts(tmem + O_COL0, tmem + 64 * (i & 1) + 8 * k,
                       desc_mn_major(v_addr + k * 16 * 128, KV_SUB_BYTES), idesc_pv, (i | k) != 0);
        umma_commit(v_empty0 + 8 * s);             // V of this stage has been read
        umma_commit(pv_done);                      // O holds pages 0..i; P of page i has been read
        if (i + 2 < n_pages) ok = issue_s(i + 2);  // overwrites the S/P buffer of page i (in order)
      }
      umma_commit(o_ready);
    }
  } else {
    // softmax: thread (warp, lane) owns query row r and tensor-memory lane r
    const int r = warp * 32 + lane;
    const int pos_r = pos0 + r;
    const int lo_r = window > 0 ? max(0, pos_r - window + 1) : 0;
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; i < n_pages && ok; ++i) {
      const uint32_t sbuf = lane_base + 64 * (i & 1);
      if (!mbar_wait(s_ready0 + 8 * (i & 1), (i >> 1) & 1)) {
        if (lane == 0) atomicExch(status, ST_SOFTMAX);
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t sr[2][32];
      tmem_ld32(sbuf, sr[0]);
      tmem_ld32(sbuf + 32, sr[1]);
      tmem_ld_wait();
      const int key0 = (first_page + i) * PAGE;
      // raw scores stay in sr; the scale (> 0) is applied to the maximum and inside the exponent.
      // Only pages that cross this row's limits are masked (warp-uniform test on the warp's rows).
      const int warp_pos_min = pos0 + warp * 32, warp_pos_max = warp_pos_min + 31;
      const bool partial = key0 + PAGE - 1 > warp_pos_min ||
                           (window > 0 && key0 < max(0, warp_pos_max - window + 1));
      if (partial) {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int key = key0 + c;
          if (key > pos_r || key < lo_r) sr[c >> 5][c & 31] = 0xff800000u;      // -inf
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};          // four short chains
#pragma unroll
      for (int c = 0; c < 64; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[c >> 5][c & 31]));
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx *= scale_log2;                            // -inf stays -inf
      const bool grow = mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY);
      if (i > 0 && __any_sync(0xffffffffu, grow)) {
        // O must hold pages 0..i-1 completely before it is rescaled
        if (!mbar_wait(pv_done, (i - 1) & 1)) {
          if (lane == 0) atomicExch(status, ST_SOFTMAX);
          ok = false;
          break;
        }
        tc_fence_after();
        const float f = grow ? ex2(m_ref - mx) : 1.f;      // 0 for a row that had seen no key
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t o[32];
          tmem_ld32(lane_base + O_COL0 + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * f);
          tmem_st32(lane_base + O_COL0 + c0, o);
        }
        tmem_st_wait();
        l *= f;
      }
      if (grow) m_ref = mx;
      const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
      uint32_t pk[32];
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        const float p0 = ex2(fmaf(__uint_as_float(sr[c >> 5][c & 31]), scale_log2, neg_m));
        const float p1 = ex2(fmaf(__uint_as_float(sr[(c + 1) >> 5][(c + 1) & 31]), scale_log2, neg_m));
        l4[(c >> 1) & 3] += p0 + p1;
        pk[c >> 1] = pack2(p0, p1);
      }
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      tmem_st32(sbuf, pk);                         // P over the first 32 columns of this S buffer
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(p_ready0 + 8 * (i & 1));
    }
    if (ok) {
      if (!mbar_wait(o_ready, 0)) {
        if (lane == 0) atomicExch(status, ST_SOFTMAX);
      } else {
        tc_fence_after();
        const float inv = 1.f / l;
        bf16 *op = out + ((size_t)(t0 + r) * nh + h) * HD;
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t o[32];
          tmem_ld32(lane_base + O_COL0 + c0, o);
          tmem_ld_wait();
          if (r < n_rows) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 v;
              v.x = pack2(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv);
              v.y = pack2(__uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
              v.z = pack2(__uint_as_float(o[j + 4]) * inv, __uint_as_float(o[j + 5]) * inv);
              v.w = pack2(__uint_as_float(o[j + 6]) * inv, __uint_as_float(o[j + 7]) * inv);
              *reinterpret_cast<uint4 *>(op + c0 + j) = v;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// q, out [T, nh*HD] bfloat16; cache [n_pages][2][nkv][64][HD] bfloat16 of one layer;
// tiles [n_tiles][4] int32 = {sequence, first token, rows (<= 128), position of row 0}.
extern "C" int g2b_attn_prefill_tc(const void *q, void *out, const void *cache, long long n_cache_pages,
                                   const int *tiles, int n_tiles, const int *page_table, int P,
                                   int T, int nh, int nkv, int hd, int page_size, int window,
                                   float scale, int *status, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (hd != HD) G2B_REFUSE("attn_prefill_tc: built for head_dim %d, got %d", HD, hd);
  if (page_size != PAGE) G2B_REFUSE("attn_prefill_tc: page size must be %d, got %d", PAGE, page_size);
  if (nkv <= 0 || nh % nkv) G2B_REFUSE("attn_prefill_tc: %d heads are not a multiple of %d kv heads", nh, nkv);
  if ((long long)n_tiles * nh > 0x7fffffffLL) G2B_REFUSE("attn_prefill_tc: %d tiles x %d heads", n_tiles, nh);
  if (!status) G2B_REFUSE("attn_prefill_tc: no status word");
  if (((uintptr_t)q | (uintptr_t)cache | (uintptr_t)out) & 15)
    G2B_REFUSE("attn_prefill_tc: q, out and the cache must be 16-byte aligned");
  if (n_cache_pages * 2 * nkv * PAGE > 0x7fffffffLL)
    G2B_REFUSE("attn_prefill_tc: the cache layer has too many rows for 32-bit copy coordinates");
  CUtensorMap mq, mkv;
  int rc = get_map(&mq, q, T, nh * HD, nh * HD, BM);
  if (rc) G2B_REFUSE("attn_prefill_tc: tensor map of q failed (%d)", rc);
  rc = get_map(&mkv, cache, n_cache_pages * 2 * nkv * PAGE, HD, HD, PAGE);
  if (rc) G2B_REFUSE("attn_prefill_tc: tensor map of the cache failed (%d)", rc);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) G2B_REFUSE("attn_prefill_tc: shared memory: %s", cudaGetErrorString(e));
    cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    configured = true;
  }
  g2b_launch(attn_prefill_tc_kernel, dim3((unsigned)n_tiles * nh), dim3(THREADS), SMEM_TOTAL, stream, mq, mkv,
             (bf16 *)out, (const int4 *)tiles, page_table, P, nh, nkv, window, scale * LOG2E, status);
  return g2b_check_launch("attn_prefill_tc");
}

extern "C" int g2b_attn_prefill_tc_tile_rows() { return BM; }
