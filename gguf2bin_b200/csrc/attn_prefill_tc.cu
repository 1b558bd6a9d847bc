// Prompt attention on the 5th-generation tensor cores: causal, grouped-query, ragged, with
// a past, over the paged bfloat16 cache (the step's own keys are already in it).
//
// Work list: tiles of 128 query rows (sequence, first token index, rows, position of the
// first row), longest first; grid (tile, query head).  Roles by warp:
//   warp 4, one thread  TMA producer: the 128 x HD query tile once, then per key page the K
//                       and V panels of (page, kv head), each as 64-column boxes with 128-byte
//                       swizzle, into a two-stage ring.
//   warp 5, one thread  MMA issuer (tcgen05.mma, cta_group::1, kind::f16):
//                         S[128 x 64]  = Q K^T      (both operands K-major)  -> tensor memory
//                         O[128 x HD] += P V        (P K-major from shared memory, V read as
//                                                    an MN-major operand: keys are its K index)
//   warps 0..3          softmax, one thread per query row: reads its row of S with tcgen05.ld,
//                       scales (log2 domain), masks (causal, window), keeps a reference maximum
//                       and a sum in float, writes P = 2^(s - m) as bfloat16 into swizzled
//                       shared memory for the second product.  O is rescaled in tensor memory
//                       only when a row's maximum has grown by more than 2^8 since its
//                       reference (the result is the same function of the scores; the factor
//                       just stays bounded), and is normalised and stored at the end.
// Per page: S MMA -> softmax -> P.V MMA; two CTAs per SM overlap each other's phases.
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
constexpr int STAGES = 2;
constexpr int SUBS = HD / 64;                       // 64-column boxes along the head dimension
constexpr int Q_SUB_BYTES = BM * 128;               // one 128 x 64 box
constexpr int Q_BYTES = SUBS * Q_SUB_BYTES;
constexpr int KV_SUB_BYTES = PAGE * 128;            // one 64 x 64 box
constexpr int KV_BYTES = SUBS * KV_SUB_BYTES;       // K (or V) of one page and kv head
constexpr int STAGE_BYTES = 2 * KV_BYTES;
constexpr int P_BYTES = BM * 128;
constexpr int BAR_OFFSET = Q_BYTES + STAGES * STAGE_BYTES + P_BYTES;
constexpr int SMEM_TOTAL = BAR_OFFSET + 128 + 1024;
constexpr int O_COL0 = 64;                          // S at columns 0..63, O from 64
constexpr int TMEM_COLS = (64 + HD) <= 128 ? 128 : 256;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.f;                 // log2 of the growth that triggers a rescale

enum { ST_PRODUCER = 11, ST_MMA = 12, ST_SOFTMAX = 13 };

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

__global__ void __launch_bounds__(THREADS)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_kv, bf16 *__restrict__ out,
                       const int4 *__restrict__ tiles, const int *__restrict__ page_table, int P,
                       int nh, int nkv, int window, float scale_log2, int *__restrict__ status) {
  pdl_launch();
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char *q_smem = smem;
  unsigned char *kv_smem = smem + Q_BYTES;
  unsigned char *p_smem = smem + Q_BYTES + STAGES * STAGE_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + BAR_OFFSET);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 8);
  const uint32_t q_full = smem_addr(bars + 0), kv_full0 = smem_addr(bars + 1);
  const uint32_t kv_empty0 = smem_addr(bars + 3), s_ready = smem_addr(bars + 5);
  const uint32_t p_ready = smem_addr(bars + 6), o_ready = smem_addr(bars + 7);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full0 + 8 * s, 1);
      mbar_init(kv_empty0 + 8 * s, 1);
    }
    mbar_init(s_ready, 1);
    mbar_init(p_ready, BM);
    mbar_init(o_ready, 1);
    mbar_init_fence();
  }
  if (warp == 5) tmem_alloc(smem_addr(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();                                   // the queries and the cache come from earlier kernels

  const int4 tile = tiles[blockIdx.x];
  const int b = tile.x, t0 = tile.y, n_rows = tile.z, pos0 = tile.w;
  const int h = blockIdx.y, kvh = h / (nh / nkv);
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
      for (int i = 0; i < n_pages; ++i) {
        const int s = i % STAGES;
        if (i >= STAGES && !mbar_wait(kv_empty0 + 8 * s, ((i / STAGES) - 1) & 1)) {
          atomicExch(status, ST_PRODUCER);
          break;
        }
        const int phys = pt[i];
        const int row_k = ((phys * 2 + 0) * nkv + kvh) * PAGE;
        const int row_v = ((phys * 2 + 1) * nkv + kvh) * PAGE;
        const uint32_t dst = smem_addr(kv_smem + s * STAGE_BYTES);
        mbar_expect_tx(kv_full0 + 8 * s, STAGE_BYTES);
#pragma unroll
        for (int sub = 0; sub < SUBS; ++sub) {
          tma_load_2d(dst + sub * KV_SUB_BYTES, &map_kv, 64 * sub, row_k, kv_full0 + 8 * s);
          tma_load_2d(dst + KV_BYTES + sub * KV_SUB_BYTES, &map_kv, 64 * sub, row_v, kv_full0 + 8 * s);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = instr_desc(BM, PAGE, false);
      constexpr uint32_t idesc_pv = instr_desc(BM, HD, true);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) atomicExch(status, ST_MMA);
      for (int i = 0; i < n_pages && ok; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(kv_full0 + 8 * s, (i / STAGES) & 1)) { atomicExch(status, ST_MMA); break; }
        tc_fence_after();
        const uint32_t k_addr = smem_addr(kv_smem + s * STAGE_BYTES), v_addr = k_addr + KV_BYTES;
        // S = Q K^T: the head dimension is the K index, 16 per MMA, 64 per box
#pragma unroll
        for (int sub = 0; sub < SUBS; ++sub)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem, desc_k_major(smem_addr(q_smem + sub * Q_SUB_BYTES)) + 2 * k,
                      desc_k_major(k_addr + sub * KV_SUB_BYTES) + 2 * k, idesc_s, (sub | k) != 0);
        umma_commit(s_ready);
        if (!mbar_wait(p_ready, i & 1)) { atomicExch(status, ST_MMA); break; }
        tc_fence_after();
        // O += P V: the keys are the K index, 16 per MMA = 16 rows of 128 bytes of the V boxes
#pragma unroll
        for (int k = 0; k < PAGE / 16; ++k)
          umma_bf16(tmem + O_COL0, desc_k_major(smem_addr(p_smem)) + 2 * k,
                    desc_mn_major(v_addr + k * 16 * 128, KV_SUB_BYTES), idesc_pv, (i | k) != 0);
        umma_commit(kv_empty0 + 8 * s);            // K and V of this stage have been read
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
      if (!mbar_wait(s_ready, i & 1)) {
        if (lane == 0) atomicExch(status, ST_SOFTMAX);
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t sr[2][32];
      tmem_ld32(lane_base, sr[0]);
      tmem_ld32(lane_base + 32, sr[1]);
      tmem_ld_wait();
      const int key0 = (first_page + i) * PAGE;
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        const int key = key0 + c;
        float v = __uint_as_float(sr[c >> 5][c & 31]) * scale_log2;
        if (key > pos_r || key < lo_r) v = -INFINITY;
        sr[c >> 5][c & 31] = __float_as_uint(v);
        mx = fmaxf(mx, v);
      }
      // s_ready(i) also means that P.V of page i-1 has completed: P may be overwritten, O is stable
      const bool grow = mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY);
      if (i > 0 && __any_sync(0xffffffffu, grow)) {
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
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      unsigned char *prow = p_smem + r * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        float p[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int c = 8 * ch + j;
          p[j] = ex2(__uint_as_float(sr[c >> 5][c & 31]) - m_use);
          l += p[j];
        }
        uint4 v;
        v.x = pack2(p[0], p[1]); v.y = pack2(p[2], p[3]);
        v.z = pack2(p[4], p[5]); v.w = pack2(p[6], p[7]);
        *reinterpret_cast<uint4 *>(prow + ((ch ^ (r & 7)) << 4)) = v;
      }
      fence_async_shared();
      tc_fence_before();
      mbar_arrive(p_ready);
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
  if (nh > 65535) G2B_REFUSE("attn_prefill_tc: %d heads", nh);
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
    configured = true;
  }
  g2b_launch(attn_prefill_tc_kernel, dim3(n_tiles, nh), dim3(THREADS), SMEM_TOTAL, stream, mq, mkv,
             (bf16 *)out, (const int4 *)tiles, page_table, P, nh, nkv, window, scale * LOG2E, status);
  return g2b_check_launch("attn_prefill_tc");
}

extern "C" int g2b_attn_prefill_tc_tile_rows() { return BM; }
