// Prompt attention on the 5th-generation tensor cores for SHORT work lists (at most two tiles
// per SM and query head: one prompt of up to about 2,000 tokens): causal, grouped-query,
// ragged, with a past, over the paged bfloat16 cache (the step's own keys are already in it).
// Same interface and results as attn_prefill_tc.cu, which keeps two CTAs on an SM and is the
// faster one when there is work for all of them (measured on a B200, 16 heads of 128: 14.3
// against 17.9 us at 1,024 tokens, 26.3 against 33.1 at 2,048, 76.8 against 67.1 at 4,096).
//
// Work list: tiles of 128 query rows (sequence, first token index, rows, position of the
// first row), longest first; one CTA per (tile, query head), numbered tile-major, one CTA on
// an SM at a time (all 512 columns of tensor memory).
//
// With few tiles the longest tile's chain of pages sets the time, and a page's softmax is a
// dependent chain of about 1,200 cycles (the exponentials alone keep the special-function unit
// busy for 512).  So a tile's pages are dealt to TWO softmax groups, even pages to one and odd
// pages to the other, each with its own MMA issuer, running maximum, sum and output
// accumulator; the two partial results of a row are merged at the end (the same function of
// the scores as one pass).  Roles by warp:
//   warp 8, one thread  TMA producer: the 128 x HD query tile once, then per key page the K
//                       and V panels of (page, kv head), each as 64-column boxes with 128-byte
//                       swizzle, into rings of four K and four V panels.
//   warps 9 and 10, one thread each: MMA issuer of group 0 and 1 (tcgen05.mma, cta_group::1,
//                       kind::f16; one thread issuing for both groups was the bottleneck):
//                         S[128 x 64]  = Q K^T      (both operands K-major) -> tensor memory,
//                                                    two S buffers per group, two pages ahead
//                         O_g[128 x HD] += P V      (P read from tensor memory, V read as an
//                                                    MN-major operand: keys are its K index)
//                       a K panel is free when its S product is done, a V panel and the S
//                       buffer (which holds P by then) when its P.V product is done: the same
//                       commit that frees V tells the group that O_g holds the page.
//   warps 0..3, 4..7    softmax groups 0 and 1: a thread owns one query row (tensor-memory
//                       lane) and all 64 keys of a page, so maxima and sums need no exchange.
//                       It scales (log2 domain), masks (causal, window), keeps a reference
//                       maximum and a sum in float, and writes P = 2^(s - m) as packed bfloat16
//                       over the first columns of the S buffer.  O_g is rescaled in tensor
//                       memory only when the row's maximum has grown by more than 2^8 since its
//                       reference (the result is the same function of the scores; the factor
//                       just stays bounded).  At the end both groups exchange (m, l) through
//                       shared memory, and each writes half of the columns of
//                       (O_0 2^(m_0 - M) + O_1 2^(m_1 - M)) / (l_0 2^(m_0 - M) + l_1 2^(m_1 - M)).
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
constexpr int GROUP_THREADS = 128;
constexpr int SOFTMAX_WARPS = 8;                    // two groups of four
constexpr int THREADS = (SOFTMAX_WARPS + 3) * 32;        // + producer, and an MMA issuer per group
constexpr int K_STAGES = 4, V_STAGES = 4;
constexpr int AHEAD = 4;                            // S products issued before the first P.V: two per group
constexpr int SUBS = HD / 64;                       // 64-column boxes along the head dimension
constexpr int Q_SUB_BYTES = BM * 128;               // one 128 x 64 box
constexpr int Q_BYTES = SUBS * Q_SUB_BYTES;
constexpr int KV_SUB_BYTES = PAGE * 128;            // one 64 x 64 box
constexpr int KV_BYTES = SUBS * KV_SUB_BYTES;       // K (or V) of one page and kv head
constexpr int K_OFFSET = Q_BYTES, V_OFFSET = K_OFFSET + K_STAGES * KV_BYTES;
constexpr int ML_OFFSET = V_OFFSET + V_STAGES * KV_BYTES;        // [2 groups][128 rows] (m, l)
constexpr int BAR_OFFSET = ML_OFFSET + 2 * BM * 8;
// one CTA per SM (it takes all of the tensor memory): at least half of an SM's shared memory
constexpr int SMEM_TOTAL = BAR_OFFSET + 512 > 115 * 1024 ? BAR_OFFSET + 512 : 115 * 1024;
static_assert(SMEM_TOTAL + 1024 <= 227 * 1024, "shared memory of an SM");
static_assert(2 * SMEM_TOTAL > 227 * 1024, "one CTA per SM");
// tensor memory: S buffers of group g at columns 64 (2 g + b), b = 0, 1; O_g at 256 + 128 g
constexpr int O_COL0 = 256, O_COLS = 128;
constexpr int TMEM_COLS = 512;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.f;                 // log2 of the growth that triggers a rescale

enum { ST_PRODUCER = 11, ST_MMA = 12, ST_SOFTMAX = 13, ST_ALIGN = 14 };
static_assert(HD <= O_COLS, "an output accumulator has 128 columns");

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// two floats at a time (one instruction of the packed kind each)
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}\n"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}\n"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}
#ifdef G2B_ATTN_TIMING
// Development aid (off unless built with -DG2B_ATTN_TIMING): cycles that the roles of CTA 0
// spend waiting and working, read back with g2b_attn_prefill_tc_timing.
__device__ unsigned long long g2b_timing[24];
#define TDECL(slot) long long tacc_##slot = 0
#define TICK(v) const long long v = clock64()
#define TOCK(slot, v) tacc_##slot += clock64() - v
#define TFLUSH(slot) if (blockIdx.x == 0) g2b_timing[slot] = (unsigned long long)tacc_##slot
#else
#define TDECL(slot)
#define TICK(v)
#define TOCK(slot, v)
#define TFLUSH(slot)
#endif
// all 256 softmax threads (barrier 1)
__device__ __forceinline__ void softmax_sync() {
  asm volatile("bar.sync 1, %0;\n" ::"n"(2 * GROUP_THREADS) : "memory");
}
// a wait of a whole warp: the same outcome for every lane (what follows is warp-wide)
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity));
}

__global__ void __launch_bounds__(THREADS, 1)
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
  float2 *ml_smem = reinterpret_cast<float2 *>(smem + ML_OFFSET);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + BAR_OFFSET);
  const uint32_t q_full = smem_addr(bars + 0);
  const uint32_t k_full0 = smem_addr(bars + 1), k_empty0 = smem_addr(bars + 1 + K_STAGES);
  const uint32_t v_full0 = smem_addr(bars + 1 + 2 * K_STAGES), v_empty0 = smem_addr(bars + 1 + 2 * K_STAGES + V_STAGES);
  constexpr int B0 = 1 + 2 * K_STAGES + 2 * V_STAGES;
  const uint32_t s_ready0 = smem_addr(bars + B0), p_ready0 = smem_addr(bars + B0 + 4);     // [group][buffer] each
  const uint32_t o_ready = smem_addr(bars + B0 + 8);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + B0 + 9);
  static_assert((B0 + 10) * 8 <= 512, "barrier slots");

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
    for (int j = 0; j < 4; ++j) {
      mbar_init(s_ready0 + 8 * j, 1);
      mbar_init(p_ready0 + 8 * j, GROUP_THREADS);
    }
    mbar_init(o_ready, 2);                       // both issuers
    mbar_init_fence();
  }
  if (warp == SOFTMAX_WARPS + 1) tmem_alloc(smem_addr(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();                                   // the queries and the cache come from earlier kernels

  const int item = blockIdx.x;                  // tile-major, longest tile first
  const int4 tile = tiles[item / nh];
  const int b = tile.x, t0 = tile.y, n_rows = tile.z, pos0 = tile.w;
  const int h = item % nh, kvh = h / (nh / nkv);
  const int first_page = window > 0 ? max(0, pos0 - window + 1) / PAGE : 0;
  const int last_page = (pos0 + n_rows - 1) / PAGE;
  const int n_pages = last_page - first_page + 1;

  if (warp == SOFTMAX_WARPS) {
    if (lane == 0 && PRODUCER_RUNS) {
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
      // in the order of use: K0 .. K3, V0, K4, V1, K5, ...
      bool ok = true;
      for (int i = 0; i < AHEAD && i < n_pages && ok; ++i) ok = load_k(i);
      for (int i = 0; i < n_pages && ok; ++i) {
        ok = load_v(i);
        if (ok && i + AHEAD < n_pages) ok = load_k(i + AHEAD);
      }
      if (!ok) atomicExch(status, ST_PRODUCER);
    }
  } else if (warp > SOFTMAX_WARPS) {
    if (lane == 0) {
      const int g = warp - (SOFTMAX_WARPS + 1);      // this issuer's group: pages i = 2 k + g
      constexpr uint32_t idesc_s = instr_desc(BM, PAGE, false);
      constexpr uint32_t idesc_pv = instr_desc(BM, HD, true);
      // descriptors once: only the start-address field (low word) changes between products
      const uint64_t dq = desc_k_major(smem_addr(q_smem)), dk = desc_k_major(smem_addr(k_smem));
      const uint64_t dv = desc_mn_major(smem_addr(v_smem), KV_SUB_BYTES);
      const uint32_t q_lo = (uint32_t)dq, q_hi = (uint32_t)(dq >> 32);
      const uint32_t k_lo = (uint32_t)dk, k_hi = (uint32_t)(dk >> 32);
      const uint32_t v_lo = (uint32_t)dv, v_hi = (uint32_t)(dv >> 32);
      TDECL(0); TDECL(1); TDECL(2); TDECL(3); TDECL(4); TDECL(5);
      TICK(t_all);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) atomicExch(status, ST_MMA);
      // S of page i into buffer (i / 2) % 2 of the group (needs K of stage i % K_STAGES)
      auto issue_s = [&](int i) -> bool {
        const int s = i % K_STAGES;
        TICK(t_k);
        if (!mbar_wait(k_full0 + 8 * s, (i / K_STAGES) & 1)) { atomicExch(status, ST_MMA); return false; }
        TOCK(1, t_k);
        tc_fence_after();
        TICK(t_is);
        const int gb = 2 * g + ((i >> 1) & 1);
        const uint32_t ks_lo = k_lo + s * (KV_BYTES >> 4), d_s = tmem + 64 * gb;
        umma_bf16_lh<false>(d_s, q_lo, q_hi, ks_lo, k_hi, idesc_s);
#pragma unroll
        for (int n = 1; n < SUBS * 4; ++n)
          umma_bf16_lh<true>(d_s, q_lo + (n / 4) * (Q_SUB_BYTES >> 4) + 2 * (n % 4), q_hi,
                             ks_lo + (n / 4) * (KV_SUB_BYTES >> 4) + 2 * (n % 4), k_hi, idesc_s);
        umma_commit(k_empty0 + 8 * s);               // the K panel is free when these are done
        umma_commit(s_ready0 + 8 * gb);
        TOCK(4, t_is);
        return true;
      };
      for (int i = g; i < AHEAD && i < n_pages && ok; i += 2) ok = issue_s(i);
      for (int i = g, k = 0; i < n_pages && ok; i += 2, ++k) {
        const int s = i % V_STAGES;
        const int gb = 2 * g + (k & 1);
        TICK(t_v);
        if (!mbar_wait(v_full0 + 8 * s, (i / V_STAGES) & 1)) { atomicExch(status, ST_MMA); break; }
        TOCK(2, t_v);
        TICK(t_p);
        if (!mbar_wait(p_ready0 + 8 * gb, (k >> 1) & 1)) { atomicExch(status, ST_MMA); break; }
        TOCK(3, t_p);
        tc_fence_after();
        TICK(t_ipv);
        // O_g += P V: the keys are the K index, 16 per MMA: 8 packed columns of P, 16 rows of V
        const uint32_t vs_lo = v_lo + s * (KV_BYTES >> 4), p_addr = tmem + 64 * gb;
#pragma unroll
        for (int kk = 0; kk < PAGE / 16; ++kk)
          umma_bf16_ts_lh(tmem + O_COL0 + O_COLS * g, p_addr + 8 * kk, vs_lo + kk * (16 * 128 >> 4), v_hi, idesc_pv,
                          kk == 0 ? (uint32_t)(k != 0) : 1u);
        // V of this stage has been read, O_g holds this page, P has been read
        umma_commit(v_empty0 + 8 * s);
        TOCK(5, t_ipv);
        if (i + AHEAD < n_pages) ok = issue_s(i + AHEAD);   // overwrites the S/P buffer of page i (in order)
      }
      umma_commit(o_ready);
      TOCK(0, t_all);
      if (g == 0) { TFLUSH(0); TFLUSH(1); TFLUSH(2); TFLUSH(3); TFLUSH(4); TFLUSH(5); }
    }
  } else {
    // softmax: group g takes the pages i = 2 k + g; this thread owns row `row` of the tile
    const int g = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const int pos = pos0 + row;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t o_base = lane_base + O_COL0 + O_COLS * g;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    TDECL(6); TDECL(7); TDECL(8); TDECL(9); TDECL(10); TDECL(11);
    TICK(t_sm);
    for (int i = g, k = 0; i < n_pages && ok; i += 2, ++k) {
      const int gb = 2 * g + (k & 1);
      const uint32_t sbuf = lane_base + 64 * gb;
      TICK(t_s);
      if (!warp_wait(s_ready0 + 8 * gb, (k >> 1) & 1)) {
        if (lane == 0) atomicExch(status, ST_SOFTMAX);
        ok = false;
        break;
      }
      TOCK(7, t_s);
      tc_fence_after();
      TICK(t_ld);
      uint32_t sr[64];                             // the row's 64 scores of this page
      tmem_ld32(sbuf, *reinterpret_cast<uint32_t(*)[32]>(&sr[0]));
      tmem_ld32(sbuf + 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[32]));
      tmem_ld_wait();
      TOCK(8, t_ld);
      TICK(t_mx);
      const int key0 = (first_page + i) * PAGE;
      // raw scores stay in sr; the scale (> 0) is applied to the maximum and inside the exponent.
      // Only pages that cross the limits of the warp's rows are masked (warp-uniform test).
      const int warp_pos_min = pos0 + (warp & 3) * 32, warp_pos_max = warp_pos_min + 31;
      const bool partial = key0 + PAGE - 1 > warp_pos_min ||
                           (window > 0 && key0 < max(0, warp_pos_max - window + 1));
      if (partial) {
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (key0 + j > pos || key0 + j < lo) sr[j] = 0xff800000u;                 // -inf
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};                  // short chains
#pragma unroll
      for (int j = 0; j < 32; ++j)
        mx4[j & 3] = max3(mx4[j & 3], __uint_as_float(sr[2 * j]), __uint_as_float(sr[2 * j + 1]));
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;  // -inf stays -inf
      TOCK(9, t_mx);
      const bool grow = mx > m + RESCALE_STEP || (m == -INFINITY && mx > -INFINITY);
      if (k > 0 && __any_sync(0xffffffffu, grow)) {
        // O_g must hold the group's pages 0..k-1 completely before it is rescaled: P.V of page
        // i - 2 is done when its V panel is released (the next release of that panel needs P of
        // a later page of this group, so the phase cannot run ahead of this wait)
        if (!warp_wait(v_empty0 + 8 * ((i - 2) % V_STAGES), ((i - 2) / V_STAGES) & 1)) {
          if (lane == 0) atomicExch(status, ST_SOFTMAX);
          ok = false;
          break;
        }
        tc_fence_after();
        const float f = grow ? ex2(m - mx) : 1.f;              // 0 for a row that had seen no key
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t o[32];
          tmem_ld32(o_base + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * f);
          tmem_st32(o_base + c0, o);
        }
        tmem_st_wait();
        l *= f;
      }
      if (grow) m = mx;
      const float neg = m == -INFINITY ? 0.f : -m;
      // two scores at a time: one packed multiply-add into the exponent, one packed addition into the sums
      TICK(t_ex);
      uint32_t pk[32];                             // packed column j: keys 2 j, 2 j + 1
      float2 l2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      const float2 sc2 = make_float2(scale_log2, scale_log2), ng2 = make_float2(neg, neg);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float2 x = fma2(make_float2(__uint_as_float(sr[2 * j]), __uint_as_float(sr[2 * j + 1])), sc2, ng2);
        const float2 pr = make_float2(ex2(x.x), ex2(x.y));
        l2[j & 1] = add2(l2[j & 1], pr);
        pk[j] = pack2(pr.x, pr.y);
      }
      l += (l2[0].x + l2[0].y) + (l2[1].x + l2[1].y);
      TOCK(10, t_ex);
      TICK(t_st);
      tmem_st32(sbuf, pk);                         // P over the first 32 columns of this S buffer
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(p_ready0 + 8 * gb);
      TOCK(11, t_st);
    }
    TOCK(6, t_sm);
#ifdef G2B_ATTN_TIMING
    if ((threadIdx.x & 127) == 0 && blockIdx.x == 0) {
      const int o = 6 + 6 * g;
      g2b_timing[o] = tacc_6; g2b_timing[o + 1] = tacc_7; g2b_timing[o + 2] = tacc_8;
      g2b_timing[o + 3] = tacc_9; g2b_timing[o + 4] = tacc_10; g2b_timing[o + 5] = tacc_11;
    }
#endif
    if (ok && !warp_wait(o_ready, 0)) {
      if (lane == 0) atomicExch(status, ST_SOFTMAX);
      ok = false;
    }
    tc_fence_after();
    // the two groups' partial results of a row: (m, l) through shared memory, O_0 and O_1 in
    // tensor memory, where both groups' warps of a lane quarter can read them
    ml_smem[g * BM + row] = make_float2(ok ? m : NAN, l);
    softmax_sync();
    const float2 other = ml_smem[(g ^ 1) * BM + row];
    if (__all_sync(0xffffffffu, ok && other.x == other.x)) {   // nothing is written after a wait that gave up
      const float m0 = g == 0 ? m : other.x, m1 = g == 0 ? other.x : m;
      const float l0 = g == 0 ? l : other.y, l1 = g == 0 ? other.y : l;
      const float mm = fmaxf(m0, m1);                          // finite for a row of the tile: it sees its own key
      const float a0 = m0 == -INFINITY ? 0.f : ex2(m0 - mm), a1 = m1 == -INFINITY ? 0.f : ex2(m1 - mm);
      const float inv = 1.f / (l0 * a0 + l1 * a1);
      const float w0 = a0 * inv, w1 = a1 * inv;
      const bool two = n_pages > 1;                            // the second group has had pages
      // group g writes columns [g HD / 2, (g + 1) HD / 2) of the row
      constexpr int HALF = HD / 2;
      bf16 *op = out + ((size_t)(t0 + row) * nh + h) * HD + g * HALF;
#pragma unroll 1
      for (int c0 = 0; c0 < HALF; c0 += 32) {
        uint32_t o0[32], o1[32];
        tmem_ld32(lane_base + O_COL0 + g * HALF + c0, o0);
        if (two) tmem_ld32(lane_base + O_COL0 + O_COLS + g * HALF + c0, o1);
        tmem_ld_wait();
        if (row < n_rows) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              v[e] = __uint_as_float(o0[j + e]) * w0;
              if (two) v[e] = fmaf(__uint_as_float(o1[j + e]), w1, v[e]);
            }
            *reinterpret_cast<uint4 *>(op + c0 + j) =
                make_uint4(pack2(v[0], v[1]), pack2(v[2], v[3]), pack2(v[4], v[5]), pack2(v[6], v[7]));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == SOFTMAX_WARPS + 1) {
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
  if (hd != HD) G2B_REFUSE("attn_prefill_tc (split): built for head_dim %d, got %d", HD, hd);
  if (page_size != PAGE) G2B_REFUSE("attn_prefill_tc (split): page size must be %d, got %d", PAGE, page_size);
  if (nkv <= 0 || nh % nkv) G2B_REFUSE("attn_prefill_tc (split): %d heads are not a multiple of %d kv heads", nh, nkv);
  if ((long long)n_tiles * nh > 0x7fffffffLL) G2B_REFUSE("attn_prefill_tc (split): %d tiles x %d heads", n_tiles, nh);
  if (!status) G2B_REFUSE("attn_prefill_tc (split): no status word");
  if (((uintptr_t)q | (uintptr_t)cache | (uintptr_t)out) & 15)
    G2B_REFUSE("attn_prefill_tc (split): q, out and the cache must be 16-byte aligned");
  if (n_cache_pages * 2 * nkv * PAGE > 0x7fffffffLL)
    G2B_REFUSE("attn_prefill_tc (split): the cache layer has too many rows for 32-bit copy coordinates");
  CUtensorMap mq, mkv;
  int rc = get_map(&mq, q, T, nh * HD, nh * HD, BM);
  if (rc) G2B_REFUSE("attn_prefill_tc (split): tensor map of q failed (%d)", rc);
  rc = get_map(&mkv, cache, n_cache_pages * 2 * nkv * PAGE, HD, HD, PAGE);
  if (rc) G2B_REFUSE("attn_prefill_tc (split): tensor map of the cache failed (%d)", rc);
  static G2bPerDevice configured;
  const int cfg_dev = g2b_current_device();
  if (cfg_dev < 0 || !configured.value[cfg_dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) G2B_REFUSE("attn_prefill_tc (split): shared memory: %s", cudaGetErrorString(e));
    cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (cfg_dev >= 0) configured.value[cfg_dev] = 1;
  }
  g2b_launch(attn_prefill_tc_kernel, dim3((unsigned)n_tiles * nh), dim3(THREADS), SMEM_TOTAL, stream, mq, mkv,
             (bf16 *)out, (const int4 *)tiles, page_table, P, nh, nkv, window, scale * LOG2E, status);
  return g2b_check_launch("attn_prefill_tc (split)");
}

extern "C" int g2b_attn_prefill_tc_tile_rows() { return BM; }


#ifdef G2B_ATTN_TIMING
// Copies the 24 counters to `out` and clears them.
extern "C" int g2b_attn_prefill_tc_timing(unsigned long long *out) {
  static unsigned long long zero[24] = {0};
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out, g2b_timing, sizeof(zero));
  cudaMemcpyToSymbol(g2b_timing, zero, sizeof(zero));
  return 0;
}
#endif
