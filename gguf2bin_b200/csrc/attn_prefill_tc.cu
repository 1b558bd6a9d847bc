// Prompt attention on the 5th-generation tensor cores: causal, grouped-query, ragged, with
// a past, over the paged bfloat16 cache (the step's own keys are already in it).
//
// Work list: tiles of 128 query rows (sequence, first token index, rows, position of the
// first row), longest first; one CTA per (tile, query head), numbered tile-major so that the
// long tiles of every head start first and the short ones fill in behind them.  Two CTAs fit
// on an SM (shared memory and tensor memory are sized for that): while one waits on its
// softmax the other's products run.  Roles by warp:
//   warp 8, one thread  TMA producer: the 128 x HD query tile once, then per key page the K
//                       and V panels of (page, kv head), each as 64-column boxes with 128-byte
//                       swizzle, into a ring of three K panels and a ring of two V panels (K is
//                       free again as soon as its S product is done, V only after P.V).
//   warp 9, one thread  MMA issuer (tcgen05.mma, cta_group::1, kind::f16):
//                         S[128 x 64]  = Q K^T      (both operands K-major)  -> tensor memory,
//                                                    two S buffers, always one page ahead
//                         O[128 x HD] += P V        (P read from tensor memory, V read as
//                                                    an MN-major operand: keys are its K index)
//   warps 0..7          softmax, 16 query rows per warp (warps w and w + 4 share a quarter of
//                       the tensor-memory lanes; each takes 16 of its 32 lanes).  S is read
//                       with the 16-lane shape whose layout is that of a warp-level product's
//                       accumulator: a thread holds two rows and, with the three other threads
//                       of its quad, all 64 keys of them, so row maxima are two shuffles.  It
//                       scales (log2 domain), masks (causal, window), keeps a reference maximum
//                       and a partial sum per row in float, and writes P = 2^(s - m) as packed
//                       bfloat16 back into the first columns of the same S buffer, where the
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
constexpr int SOFTMAX_WARPS = 8;
constexpr int THREADS = (SOFTMAX_WARPS + 2) * 32;
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
__device__ unsigned long long g2b_timing[16];
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

#ifndef G2B_ATTN_MINBLOCKS
#define G2B_ATTN_MINBLOCKS 2
#endif
__global__ void __launch_bounds__(THREADS, G2B_ATTN_MINBLOCKS)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_kv, bf16 *__restrict__ out,
                       const int4 *__restrict__ tiles, const int *__restrict__ page_table, int P,
                       int nh, int nkv, int window, float scale_log2, int first_wave,
                       int *__restrict__ status) {
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
  const uint32_t o_ready = smem_addr(bars + 15);
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
      mbar_init(p_ready0 + 8 * j, SOFTMAX_WARPS * 32);
    }
    mbar_init(o_ready, 1);
    mbar_init_fence();
  }
  if (warp == SOFTMAX_WARPS + 1) tmem_alloc(smem_addr(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();                                   // the queries and the cache come from earlier kernels

  // CTA -> (tile, head).  Items are numbered tile-major, longest tile first.  The first wave
  // (one CTA on every SM) takes them from the long end.  When everything fits in two waves the
  // second CTAs of the SMs take the rest from the short end, so that the longest tiles share
  // their SM with the shortest; with more waves the rest follows longest first.
  const int n_items = gridDim.x;
  int item = blockIdx.x;
  if (item >= first_wave && n_items <= 2 * first_wave) item = n_items - 1 - (item - first_wave);
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
      // in the order of use: K0, K1, V0, K2, V1, K3, ...
      bool ok = load_k(0);
      for (int i = 0; i < n_pages && ok; ++i) {
        if (i + 1 < n_pages) ok = load_k(i + 1);
        if (ok) ok = load_v(i);
      }
      if (!ok) atomicExch(status, ST_PRODUCER);
    }
  } else if (warp == SOFTMAX_WARPS + 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = instr_desc(BM, PAGE, false);
      constexpr uint32_t idesc_pv = instr_desc(BM, HD, true);
      // descriptors once: only the start-address field (low word) changes between products
      const uint64_t dq = desc_k_major(smem_addr(q_smem)), dk = desc_k_major(smem_addr(k_smem));
      const uint64_t dv = desc_mn_major(smem_addr(v_smem), KV_SUB_BYTES);
      const uint32_t q_lo = (uint32_t)dq, q_hi = (uint32_t)(dq >> 32);
      const uint32_t k_lo = (uint32_t)dk, k_hi = (uint32_t)(dk >> 32);
      const uint32_t v_lo = (uint32_t)dv, v_hi = (uint32_t)(dv >> 32);
      TDECL(0); TDECL(1); TDECL(2); TDECL(3); TDECL(9); TDECL(10); TDECL(11);
      TICK(t_all);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) atomicExch(status, ST_MMA);
      // S of page i into S buffer i % 2 (needs K of stage i % K_STAGES).  The softmax warps see
      // its completion and pass it on to the producer (the K panel is free then).
      auto issue_s = [&](int i) -> bool {
        const int s = i % K_STAGES;
        TICK(t_k);
        if (!mbar_wait(k_full0 + 8 * s, (i / K_STAGES) & 1)) { atomicExch(status, ST_MMA); return false; }
        TOCK(1, t_k);
        tc_fence_after();
        const uint32_t ks_lo = k_lo + s * (KV_BYTES >> 4), d_s = tmem + 64 * (i & 1);
        TICK(t_is);
        umma_bf16_lh<false>(d_s, q_lo, q_hi, ks_lo, k_hi, idesc_s);
#pragma unroll
        for (int n = 1; n < SUBS * 4; ++n)
          umma_bf16_lh<true>(d_s, q_lo + (n / 4) * (Q_SUB_BYTES >> 4) + 2 * (n % 4), q_hi,
                             ks_lo + (n / 4) * (KV_SUB_BYTES >> 4) + 2 * (n % 4), k_hi, idesc_s);
        TOCK(9, t_is);
        TICK(t_cs);
        umma_commit(s_ready0 + 8 * (i & 1));
        TOCK(10, t_cs);
        return true;
      };
      if (ok) ok = issue_s(0);
      if (ok && n_pages > 1) ok = issue_s(1);
      for (int i = 0; i < n_pages && ok; ++i) {
        const int s = i % V_STAGES;
        TICK(t_v);
        if (!mbar_wait(v_full0 + 8 * s, (i / V_STAGES) & 1)) { atomicExch(status, ST_MMA); break; }
        TOCK(2, t_v);
        TICK(t_p);
        if (!mbar_wait(p_ready0 + 8 * (i & 1), (i >> 1) & 1)) { atomicExch(status, ST_MMA); break; }
        TOCK(3, t_p);
        tc_fence_after();
        // O += P V: the keys are the K index, 16 per MMA: 8 packed columns of P, 16 rows of V
        const uint32_t vs_lo = v_lo + s * (KV_BYTES >> 4), p_addr = tmem + 64 * (i & 1);
        TICK(t_ipv);
#pragma unroll
        for (int k = 0; k < PAGE / 16; ++k)
          umma_bf16_ts_lh(tmem + O_COL0, p_addr + 8 * k, vs_lo + k * (16 * 128 >> 4), v_hi, idesc_pv,
                          k == 0 ? (uint32_t)(i != 0) : 1u);
        TOCK(11, t_ipv);
        // V of this stage has been read, O holds pages 0..i, P of page i has been read
        umma_commit(v_empty0 + 8 * s);
        if (i + 2 < n_pages) ok = issue_s(i + 2);  // overwrites the S/P buffer of page i (in order)
      }
      umma_commit(o_ready);
      TOCK(0, t_all);
      TFLUSH(0); TFLUSH(1); TFLUSH(2); TFLUSH(3); TFLUSH(9); TFLUSH(10); TFLUSH(11);
    }
  } else {
    // softmax: this warp owns rows row0 .. row0 + 15 (tensor-memory lanes of the same numbers);
    // the thread holds rows rA = row0 + g and rB = rA + 8, keys 8j + 2c, 8j + 2c + 1 of a page
    const int g = lane >> 2, c = lane & 3;
    const int row0 = (warp & 3) * 32 + (warp >> 2) * 16;
    const int rA = row0 + g, rB = rA + 8;
    const int pos_a = pos0 + rA, pos_b = pos0 + rB;
    const int lo_a = window > 0 ? max(0, pos_a - window + 1) : 0;
    const int lo_b = window > 0 ? max(0, pos_b - window + 1) : 0;
    const uint32_t lane_base = tmem + ((uint32_t)row0 << 16);
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;      // l: this thread's keys only
    bool ok = true;
    TDECL(4); TDECL(5); TDECL(6); TDECL(7); TDECL(12); TDECL(13);
    TICK(t_sm);
    for (int i = 0; i < n_pages && ok; ++i) {
      const uint32_t sbuf = lane_base + 64 * (i & 1);
      TICK(t_s);
      if (!mbar_wait(s_ready0 + 8 * (i & 1), (i >> 1) & 1)) {
        if (lane == 0) atomicExch(status, ST_SOFTMAX);
        ok = false;
        break;
      }
      TOCK(5, t_s);
      if (threadIdx.x == 0) mbar_arrive(k_empty0 + 8 * (i % K_STAGES));       // S of page i is done: K is free
      tc_fence_after();
      uint32_t sr[32];                             // [4j + 2s + e]: row (s ? rB : rA), key 8j + 2c + e
      TICK(t_ld);
      tmem_ld_16x256b_x8(sbuf, sr);
      tmem_ld_wait();
      TOCK(6, t_ld);
      const int key0 = (first_page + i) * PAGE;
      TICK(t_mx);
      // raw scores stay in sr; the scale (> 0) is applied to the maximum and inside the exponent.
      // Only pages that cross the limits of the warp's rows are masked (warp-uniform test).
      const int warp_pos_min = pos0 + row0, warp_pos_max = warp_pos_min + 15;
      const bool partial = key0 + PAGE - 1 > warp_pos_min ||
                           (window > 0 && key0 < max(0, warp_pos_max - window + 1));
      if (partial) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int key = key0 + 8 * j + 2 * c + e;
            if (key > pos_a || key < lo_a) sr[4 * j + e] = 0xff800000u;           // -inf
            if (key > pos_b || key < lo_b) sr[4 * j + 2 + e] = 0xff800000u;
          }
      }
      float mxa[2] = {-INFINITY, -INFINITY}, mxb[2] = {-INFINITY, -INFINITY};       // short chains
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        mxa[j & 1] = max3(mxa[j & 1], __uint_as_float(sr[4 * j]), __uint_as_float(sr[4 * j + 1]));
        mxb[j & 1] = max3(mxb[j & 1], __uint_as_float(sr[4 * j + 2]), __uint_as_float(sr[4 * j + 3]));
      }
      float mx_a = fmaxf(mxa[0], mxa[1]), mx_b = fmaxf(mxb[0], mxb[1]);
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      mx_a *= scale_log2;                          // -inf stays -inf
      mx_b *= scale_log2;
      TOCK(12, t_mx);
      const bool grow_a = mx_a > m_a + RESCALE_STEP || (m_a == -INFINITY && mx_a > -INFINITY);
      const bool grow_b = mx_b > m_b + RESCALE_STEP || (m_b == -INFINITY && mx_b > -INFINITY);
      if (i > 0 && __any_sync(0xffffffffu, grow_a || grow_b)) {
        // O must hold pages 0..i-1 completely before it is rescaled: P.V of page i-1 is done when
        // its V panel is released (the next release of that panel needs P of page i+1, so the
        // phase cannot run ahead of this wait)
        if (!mbar_wait(v_empty0 + 8 * ((i - 1) % V_STAGES), ((i - 1) / V_STAGES) & 1)) {
          if (lane == 0) atomicExch(status, ST_SOFTMAX);
          ok = false;
          break;
        }
        tc_fence_after();
        const float f_a = grow_a ? ex2(m_a - mx_a) : 1.f;      // 0 for a row that had seen no key
        const float f_b = grow_b ? ex2(m_b - mx_b) : 1.f;
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 64) {
          uint32_t o[32];
          tmem_ld_16x256b_x8(lane_base + O_COL0 + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            o[4 * j] = __float_as_uint(__uint_as_float(o[4 * j]) * f_a);
            o[4 * j + 1] = __float_as_uint(__uint_as_float(o[4 * j + 1]) * f_a);
            o[4 * j + 2] = __float_as_uint(__uint_as_float(o[4 * j + 2]) * f_b);
            o[4 * j + 3] = __float_as_uint(__uint_as_float(o[4 * j + 3]) * f_b);
          }
          tmem_st_16x256b_x8(lane_base + O_COL0 + c0, o);
        }
        tmem_st_wait();
        l_a *= f_a;
        l_b *= f_b;
      }
      if (grow_a) m_a = mx_a;
      if (grow_b) m_b = mx_b;
      const float neg_a = m_a == -INFINITY ? 0.f : -m_a;
      const float neg_b = m_b == -INFINITY ? 0.f : -m_b;
      TICK(t_ex);
      uint32_t pk[16];                             // [2j + s]: row (s ? rB : rA), packed column 4j + c
      // two scores at a time: one packed multiply-add into the exponent, one packed addition into the sums
      float2 la2 = make_float2(0.f, 0.f), lb2 = make_float2(0.f, 0.f);
      const float2 sc2 = make_float2(scale_log2, scale_log2);
      const float2 na2 = make_float2(neg_a, neg_a), nb2 = make_float2(neg_b, neg_b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 xa = fma2(make_float2(__uint_as_float(sr[4 * j]), __uint_as_float(sr[4 * j + 1])), sc2, na2);
        const float2 xb = fma2(make_float2(__uint_as_float(sr[4 * j + 2]), __uint_as_float(sr[4 * j + 3])), sc2, nb2);
        const float2 pa = make_float2(ex2(xa.x), ex2(xa.y)), pb = make_float2(ex2(xb.x), ex2(xb.y));
        la2 = add2(la2, pa);
        lb2 = add2(lb2, pb);
        pk[2 * j] = pack2(pa.x, pa.y);
        pk[2 * j + 1] = pack2(pb.x, pb.y);
      }
      l_a += la2.x + la2.y;
      l_b += lb2.x + lb2.y;
      TOCK(13, t_ex);
      TICK(t_st);
      tmem_st_16x128b_x8(sbuf, pk);                // P over the first 32 columns of this S buffer
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(p_ready0 + 8 * (i & 1));
      TOCK(7, t_st);
    }
    TOCK(4, t_sm);
    if (threadIdx.x == 0) { TFLUSH(4); TFLUSH(5); TFLUSH(6); TFLUSH(7); TFLUSH(12); TFLUSH(13); }
    if (ok) {
      if (!mbar_wait(o_ready, 0)) {
        if (lane == 0) atomicExch(status, ST_SOFTMAX);
      } else {
        tc_fence_after();
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
        const float inv_a = 1.f / l_a, inv_b = 1.f / l_b;
        bf16 *op_a = out + ((size_t)(t0 + rA) * nh + h) * HD + 2 * c;
        bf16 *op_b = out + ((size_t)(t0 + rB) * nh + h) * HD + 2 * c;
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 64) {
          uint32_t o[32];
          tmem_ld_16x256b_x8(lane_base + O_COL0 + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (rA < n_rows)
              *reinterpret_cast<uint32_t *>(op_a + c0 + 8 * j) =
                  pack2(__uint_as_float(o[4 * j]) * inv_a, __uint_as_float(o[4 * j + 1]) * inv_a);
            if (rB < n_rows)
              *reinterpret_cast<uint32_t *>(op_b + c0 + 8 * j) =
                  pack2(__uint_as_float(o[4 * j + 2]) * inv_b, __uint_as_float(o[4 * j + 3]) * inv_b);
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
  static G2bPerDevice configured;                      // holds the device's SM count once it is set up
  const int cfg_dev = g2b_current_device();
  int n_sms = cfg_dev >= 0 ? configured.value[cfg_dev] : 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) G2B_REFUSE("attn_prefill_tc: shared memory: %s", cudaGetErrorString(e));
    cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (cfg_dev >= 0) configured.value[cfg_dev] = n_sms;
  }
  g2b_launch(attn_prefill_tc_kernel, dim3((unsigned)n_tiles * nh), dim3(THREADS), SMEM_TOTAL, stream, mq, mkv,
             (bf16 *)out, (const int4 *)tiles, page_table, P, nh, nkv, window, scale * LOG2E, n_sms, status);
  return g2b_check_launch("attn_prefill_tc");
}

extern "C" int g2b_attn_prefill_tc_tile_rows() { return BM; }

#ifdef G2B_ATTN_TIMING
// Copies the 16 counters to `out` and clears them.
extern "C" int g2b_attn_prefill_tc_timing(unsigned long long *out) {
  static unsigned long long zero[16] = {0};
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out, g2b_timing, sizeof(zero));
  cudaMemcpyToSymbol(g2b_timing, zero, sizeof(zero));
  return 0;
}
#endif
