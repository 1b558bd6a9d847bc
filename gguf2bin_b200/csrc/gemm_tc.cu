// Matrix product for many rows (prompts) on the 5th-generation tensor cores:
//   C[M,N] = A[M,K] * W[N,K]^T, bfloat16 operands, float accumulation in tensor memory.
//
// One CTA computes a 128 x BN tile of C.  Roles by warp:
//   warp 4, one thread   TMA producer: for every 64-wide block of K, two tiled bulk copies
//                        (cp.async.bulk.tensor.2d, 128-byte swizzle) bring A[128 x 64] and
//                        W[BN x 64] into a ring of shared-memory stages and signal the
//                        stage's "full" mbarrier with their byte count.  No multicast.
//   warp 5, one thread   MMA issuer: waits for "full", issues four tcgen05.mma
//                        (cta_group::1, kind::f16, M=128, N=BN, K=16) whose operands are
//                        shared-memory descriptors (K-major, SWIZZLE_128B, 1024 bytes between
//                        8-row groups) and whose accumulator is BN columns of tensor memory;
//                        tcgen05.commit frees the stage ("empty") and, after the last block,
//                        signals "accumulator ready".  Warp 5 also allocates and frees the
//                        tensor memory.
//   warps 0..3           epilogue: each warp reads its 32 lanes of the accumulator with
//                        tcgen05.ld (32 columns at a time) and writes C: store (bfloat16 or
//                        float), add into a float matrix (the residual stream), or the SiLU
//                        gate on a fused gate/up matrix whose rows alternate 8 gates / 8 ups
//                        (src/l3_math.c:57-62, src/l5_model.c:594-595 of AnonymoDGH/gguf2bin).
// Rows and columns past M, N and K are zero-filled by the TMA unit on load and masked on store.
//
// Every wait (mbarrier) gives up after a bounded number of polls: the thread records a
// code in `*status`, all roles fall through to the common exit, the tensor memory is freed
// and the kernel returns; the host reads `*status` (0 = fine).
#include "common.cuh"
#include "tc_common.cuh"

G2B_DEFINE_LAST_ERROR

using namespace tc;

constexpr int BM = 128;
constexpr int BK = 64;                      // 64 bf16 = 128 bytes = one swizzle row
constexpr int THREADS = 192;

enum { EPI_STORE_BF16 = 0, EPI_STORE_F32 = 1, EPI_ACCUM_F32 = 2, EPI_SWIGLU_BF16 = 3 };
enum { ST_OK = 0, ST_PRODUCER_TIMEOUT = 1, ST_MMA_TIMEOUT = 2, ST_EPILOGUE_TIMEOUT = 3 };

__device__ __forceinline__ uint32_t pack2(uint32_t lo, uint32_t hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(lo), __uint_as_float(hi));
  return *reinterpret_cast<uint32_t *>(&v);
}

__device__ __forceinline__ uint32_t pack2f(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

// Instruction descriptor of a product with M = 128, N = n, both operands K-major.
__host__ __device__ constexpr uint32_t idesc_n(int n) { return instr_desc(BM, n, false); }

template <int BN, int STAGES> struct Smem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BARRIER_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BARRIER_OFFSET + 128 + 1024;   // barriers + tmem slot + alignment slack
};

// Epilogue of one 128 x BN tile by one of the four epilogue warps: warp w owns accumulator
// lanes (rows) 32w .. 32w+31 and reads them 32 columns at a time.  `scr` is 32 x 33 floats of
// shared memory of this warp (used by the float outputs to turn rows into coalesced stores).
template <int BN, int EPI>
__device__ __forceinline__ void epilogue_tile(uint32_t tmem, float *scr, void *__restrict__ Cv, int m0, int n0,
                                              int M, int N, int ldc, int warp, int lane) {
      const int row = m0 + warp * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        const int n = n0 + c0;
        if (EPI == EPI_STORE_F32 || EPI == EPI_ACCUM_F32) {
          // through shared memory, so that a warp touches 128 contiguous bytes of one row of
          // C at a time (the operand stages are free: every MMA has completed)
          if (n >= N) continue;                              // uniform over the warp
#pragma unroll
          for (int j = 0; j < 32; ++j) scr[lane * 33 + j] = __uint_as_float(r[j]);
          __syncwarp();
          const bool col_ok = n + lane < N;
          float *cbase = (float *)Cv + (size_t)(m0 + warp * 32) * ldc + n + lane;
#pragma unroll 8
          for (int rr = 0; rr < 32; ++rr) {
            if (col_ok && m0 + warp * 32 + rr < M) {
              float *p = cbase + (size_t)rr * ldc;
              const float v = scr[rr * 33 + lane];
              // one thread adds to an element once per launch, so the reduction (no value
              // comes back, nothing waits for the old one) gives the same sum as load-add-store
              if (EPI == EPI_ACCUM_F32) atomicAdd(p, v);
              else *p = v;
            }
          }
          __syncwarp();
          continue;
        }
        if (row >= M || n >= N) continue;
        if (EPI == EPI_SWIGLU_BF16) {
          // columns 16b .. 16b+7 are gates, 16b+8 .. 16b+15 the ups of the same outputs
          bf16 *dst = (bf16 *)Cv + (size_t)row * ldc + (n >> 1);
          float h[16];
#pragma unroll
          for (int blk = 0; blk < 2; ++blk)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float gate = __uint_as_float(r[16 * blk + j]);
              const float up = __uint_as_float(r[16 * blk + 8 + j]);
              h[8 * blk + j] = __fdividef(gate, 1.f + __expf(-gate)) * up;
            }
          if (n + 32 <= N && ((((uintptr_t)dst) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 16; j += 8) {
              uint4 v;
              v.x = pack2f(h[j], h[j + 1]); v.y = pack2f(h[j + 2], h[j + 3]);
              v.z = pack2f(h[j + 4], h[j + 5]); v.w = pack2f(h[j + 6], h[j + 7]);
              *reinterpret_cast<uint4 *>(dst + j) = v;
            }
          } else {
#pragma unroll
            for (int blk = 0; blk < 2; ++blk)
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (n + 16 * blk + 8 + j < N) dst[8 * blk + j] = __float2bfloat16_rn(h[8 * blk + j]);
          }
        } else if (EPI == EPI_STORE_BF16) {
          bf16 *dst = (bf16 *)Cv + (size_t)row * ldc + n;
          if (n + 32 <= N && ((((uintptr_t)dst) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 v;
              v.x = pack2(r[j], r[j + 1]); v.y = pack2(r[j + 2], r[j + 3]);
              v.z = pack2(r[j + 4], r[j + 5]); v.w = pack2(r[j + 6], r[j + 7]);
              *reinterpret_cast<uint4 *>(dst + j) = v;
            }
          } else {
            for (int j = 0; j < 32 && n + j < N; ++j) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
          }
        }
      }
}

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               void *__restrict__ Cv, int M, int N, int K, int ldc, int *__restrict__ status) {
  pdl_launch();
  extern __shared__ unsigned char smem_raw[];
  using S = Smem<BN, STAGES>;
  // 1024-byte alignment: the swizzle pattern is a function of address bits 4..9
  unsigned char *smem = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + S::BARRIER_OFFSET);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 1);
  const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + STAGES);
  const uint32_t acc_bar = smem_addr(bars + 2 * STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int nkb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                     smem_addr(tmem_slot)), "r"((uint32_t)BN));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  pdl_wait();                  // barriers and tensor memory are set up; now the inputs are needed

  if (warp == 4) {
    if (lane == 0 && PRODUCER_RUNS) {
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % STAGES;
        if (kb >= STAGES && !mbar_wait(empty0 + 8 * s, ((kb / STAGES) - 1) & 1)) {
          atomicExch(status, ST_PRODUCER_TIMEOUT);
          break;
        }
        const uint32_t a_dst = smem_addr(smem + s * S::STAGE_BYTES);
        mbar_expect_tx(full0 + 8 * s, S::STAGE_BYTES);
        tma_load_2d(a_dst, &map_a, kb * BK, m0, full0 + 8 * s);
        tma_load_2d(a_dst + S::A_BYTES, &map_w, kb * BK, n0, full0 + 8 * s);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_n(BN);
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % STAGES;
        if (!mbar_wait(full0 + 8 * s, (kb / STAGES) & 1)) {
          atomicExch(status, ST_MMA_TIMEOUT);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t a_addr = smem_addr(smem + s * S::STAGE_BYTES);
        const uint64_t adesc = desc_k_major(a_addr), bdesc = desc_k_major(a_addr + S::A_BYTES);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)            // 16 bf16 = 32 bytes = 2 descriptor units
          umma_bf16(tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
        umma_commit(empty0 + 8 * s);                 // the stage is free once these MMAs have read it
      }
      umma_commit(acc_bar);                          // all MMAs issued so far have completed
    }
  } else {
    // epilogue: warp w owns accumulator lanes (rows) 32w .. 32w+31
    if (!mbar_wait(acc_bar, 0)) {
      if (lane == 0) atomicExch(status, ST_EPILOGUE_TIMEOUT);
    } else {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      epilogue_tile<BN, EPI>(tmem, reinterpret_cast<float *>(smem) + warp * (32 * 33), Cv, m0, n0, M, N, ldc, warp, lane);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"((uint32_t)BN));
  }
}

// Epilogue of one 128 x BN tile through shared memory and tile stores.  Warp w owns rows
// 32w .. 32w+31; a thread owns one row.  Per box of 128 bytes per row (64 bfloat16 or 32 float
// outputs) the thread writes its row into a 32 x 128-byte staging buffer of its warp in the
// 128-byte swizzle (16-byte chunk c of row r at chunk c ^ (r % 8): conflict-free), and lane 0
// hands the box to the bulk-copy unit, which writes whole rows of C and clips at M and N; for
// the accumulating epilogue it adds instead (one contributor per element and launch, so the
// sum does not depend on any order).  Two staging buffers per warp: the copy of one box runs
// while the next is filled.  The accumulator loads run one chunk ahead of their use.
// `box` counts the boxes this warp has issued so far (selects the buffer).
// One chunk of 32 accumulator columns (`v`, chunk `c` of the tile) on its way to C: see below.
template <int EPI>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&v)[32], int c, unsigned char *stage,
                                               const CUtensorMap *map_c, int y, int n0, int M, int N, int lane,
                                               uint32_t &box) {
  // which 16-byte chunks of the row this accumulator chunk fills, and whether it completes a box
  constexpr int PER_BOX = EPI == EPI_SWIGLU_BF16 ? 4 : (EPI == EPI_STORE_BF16 ? 2 : 1);
  const int part = c % PER_BOX;
  if (part == 0) {
    // the buffer's previous box (two boxes ago) must have been read
    if (lane == 0) bulk_wait_read<1>();
    __syncwarp();
  }
  unsigned char *buf = stage + (box & 1) * 4096;
  const uint32_t row_addr = smem_addr(buf) + lane * 128;
  auto put = [&](int chunk, uint4 val) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(row_addr + ((chunk ^ (lane & 7)) << 4)),
                 "r"(val.x), "r"(val.y), "r"(val.z), "r"(val.w) : "memory");
  };
  if (EPI == EPI_STORE_F32 || EPI == EPI_ACCUM_F32) {
#pragma unroll
    for (int j = 0; j < 8; ++j) put(j, make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
  } else if (EPI == EPI_STORE_BF16) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      put(4 * part + j, make_uint4(pack2(v[8 * j], v[8 * j + 1]), pack2(v[8 * j + 2], v[8 * j + 3]),
                                   pack2(v[8 * j + 4], v[8 * j + 5]), pack2(v[8 * j + 6], v[8 * j + 7])));
  } else {
    // columns 16b .. 16b+7 are gates, 16b+8 .. 16b+15 the ups of the same outputs
    float h[16];
#pragma unroll
    for (int blk = 0; blk < 2; ++blk)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gate = __uint_as_float(v[16 * blk + j]);
        const float up = __uint_as_float(v[16 * blk + 8 + j]);
        h[8 * blk + j] = __fdividef(gate, 1.f + __expf(-gate)) * up;
      }
#pragma unroll
    for (int j = 0; j < 2; ++j)
      put(2 * part + j, make_uint4(pack2f(h[8 * j], h[8 * j + 1]), pack2f(h[8 * j + 2], h[8 * j + 3]),
                                   pack2f(h[8 * j + 4], h[8 * j + 5]), pack2f(h[8 * j + 6], h[8 * j + 7])));
  }
  if (part == PER_BOX - 1) {
    fence_async_shared();
    __syncwarp();
    if (lane == 0) {
      const int first_col = n0 + 32 * (c - part);            // accumulator column of the box
      if (first_col < N && y < M) {                          // a box wholly outside C is not issued
        const int x = EPI == EPI_SWIGLU_BF16 ? first_col >> 1 : first_col;
        if (EPI == EPI_ACCUM_F32) tma_reduce_add_2d(map_c, smem_addr(buf), x, y);
        else tma_store_2d(map_c, smem_addr(buf), x, y);
      }
      bulk_commit();                                        // an empty group keeps the count in step
    }
    ++box;
  }
}

template <int BN, int EPI>
__device__ __forceinline__ void epilogue_tile_bulk(uint32_t tmem, unsigned char *stage, const CUtensorMap *map_c,
                                                   int m0, int n0, int M, int N, int warp, int lane,
                                                   uint32_t &box) {
  constexpr int CHUNKS = BN / 32;
  const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
  const int y = m0 + warp * 32;
  uint32_t r[2][32];
  tmem_ld32(lane_addr, r[0]);
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
    if (c + 1 < CHUNKS) tmem_ld32(lane_addr + 32 * (c + 1), r[(c + 1) & 1]);
    epilogue_chunk<EPI>(r[c & 1], c, stage, map_c, y, n0, M, N, lane, box);
  }
}

// ---- K in parts over a cluster ---------------------------------------------------------------
// With fewer tiles than half the SMs, the CTAs of a cluster take the same tile and one part of
// K each.  The tile's chunks of 32 columns are dealt out to the ranks in contiguous ranges
// (whole boxes of the output): a rank keeps its own chunks in tensor memory, lays the others
// out in its ring of stages (free once its products are done) as [chunk][128 rows][32 floats],
// and after a cluster barrier sends every other rank that one's chunks with one bulk copy
// through the cluster's window, counted on a barrier of the receiver.  Then it adds the parts
// of its own chunks in rank order (the sum does not depend on timing) and sends them through
// the ordinary epilogue.  The first chunk of rank q of S: PER_BOX * ((CHUNKS / PER_BOX) * q / S).
constexpr int PART_CHUNK_BYTES = BM * 128;          // one chunk of a tile: 128 rows of 32 floats
__host__ __device__ constexpr int chunks_per_box(int epi) {
  return epi == EPI_SWIGLU_BF16 ? 4 : (epi == EPI_STORE_BF16 ? 2 : 1);
}
template <int BN, int EPI> __host__ __device__ constexpr int part_chunk_lo(int q, int S) {
  return chunks_per_box(EPI) * (((BN / 32) / chunks_per_box(EPI)) * q / S);
}
// whether S parts fit tiles bn wide: every rank owns a box, and the chunks of the others plus
// what a rank receives fit the ring
static bool parts_fit(int bn, int epi, int S, int nkb, int ring_bytes) {
  const int per_box = chunks_per_box(epi), chunks = bn / 32;
  if (S < 1 || S > 4 || chunks / per_box < S || nkb < S) return false;
  for (int q = 0; q < S; ++q) {
    const int own = per_box * ((chunks / per_box) * (q + 1) / S) - per_box * ((chunks / per_box) * q / S);
    if ((chunks - own + (S - 1) * own) * PART_CHUNK_BYTES > ring_bytes) return false;
  }
  return true;
}

// the chunks of the other ranks into the ring (epilogue warps, after the tile's products)
template <int BN, int EPI>
__device__ __forceinline__ void parts_lay_out(uint32_t tmem, unsigned char *ring, int warp, int lane, int rank, int S) {
  constexpr int CHUNKS = BN / 32;
  const int own_lo = part_chunk_lo<BN, EPI>(rank, S), own_hi = part_chunk_lo<BN, EPI>(rank + 1, S);
  const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
  for (int c = 0; c < CHUNKS; ++c) {
    if (c >= own_lo && c < own_hi) continue;
    uint32_t r[32];
    tmem_ld32(lane_addr + 32 * c, r);
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
    const int slot = c < own_lo ? c : c - (own_hi - own_lo);
    const uint32_t row_addr = smem_addr(ring) + slot * PART_CHUNK_BYTES + (warp * 32 + lane) * 128;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(row_addr + ((j ^ (lane & 7)) << 4)),
                   "r"(r[4 * j]), "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3]) : "memory");
  }
}
// one thread: this rank's copies to the others (after the cluster barrier)
template <int BN, int EPI>
__device__ __forceinline__ void parts_send(unsigned char *ring, uint32_t part_bar, int rank, int S) {
  constexpr int CHUNKS = BN / 32;
  const int own_lo = part_chunk_lo<BN, EPI>(rank, S), own_n = part_chunk_lo<BN, EPI>(rank + 1, S) - own_lo;
  for (int q = 0; q < S; ++q) {
    if (q == rank) continue;
    const int q_lo = part_chunk_lo<BN, EPI>(q, S), q_n = part_chunk_lo<BN, EPI>(q + 1, S) - q_lo;
    if (q_n <= 0) continue;
    const int slot = q_lo < own_lo ? q_lo : q_lo - own_n;              // where q's chunks lie in my ring
    // in q's ring: after the chunks it laid out itself, one range per sender in rank order
    const uint32_t dst = smem_addr(ring) + (uint32_t)((CHUNKS - q_n) + (rank < q ? rank : rank - 1) * q_n) * PART_CHUNK_BYTES;
    asm volatile(
        "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
        ::"r"(map_to_cta(dst, (uint32_t)q)), "r"(smem_addr(ring) + (uint32_t)slot * PART_CHUNK_BYTES),
          "r"((uint32_t)q_n * PART_CHUNK_BYTES), "r"(map_to_cta(part_bar, (uint32_t)q))
        : "memory");
  }
}
// this rank's chunks: own part from tensor memory, the others' from the ring, added in rank order
template <int BN, int EPI>
__device__ __forceinline__ void parts_finish(uint32_t tmem, const unsigned char *ring, unsigned char *stage,
                                             const CUtensorMap *map_c, int m0, int n0, int M, int N, int warp,
                                             int lane, uint32_t &box, int rank, int S) {
  constexpr int CHUNKS = BN / 32;
  const int own_lo = part_chunk_lo<BN, EPI>(rank, S), own_n = part_chunk_lo<BN, EPI>(rank + 1, S) - own_lo;
  const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
  const uint32_t recv0 = smem_addr(ring) + (uint32_t)(CHUNKS - own_n) * PART_CHUNK_BYTES + (warp * 32 + lane) * 128;
  const int y = m0 + warp * 32;
#pragma unroll 1
  for (int i = 0; i < own_n; ++i) {
    uint32_t mine[32], v[32];
    tmem_ld32(lane_addr + 32 * (own_lo + i), mine);
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll 1
    for (int p = 0; p < S; ++p) {
      if (p == rank) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          v[j] = p == 0 ? mine[j] : __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(mine[j]));
      } else {
        const uint32_t src = recv0 + (uint32_t)((p < rank ? p : p - 1) * own_n + i) * PART_CHUNK_BYTES;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 t;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];\n" : "=r"(t.x), "=r"(t.y), "=r"(t.z), "=r"(t.w)
                       : "r"(src + ((j ^ (lane & 7)) << 4)) : "memory");
          const uint32_t tt[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
          for (int e = 0; e < 4; ++e)
            v[4 * j + e] = p == 0 ? tt[e] : __float_as_uint(__uint_as_float(v[4 * j + e]) + __uint_as_float(tt[e]));
        }
      }
    }
    epilogue_chunk<EPI>(v, own_lo + i, stage, map_c, y, n0, M, N, lane, box);
  }
}

// The order in which a persistent grid walks over the tiles of C.  Plainly down the rows of a
// column of tiles and then on to the next column, every column of tiles reads all of A again;
// that is free while A stays in the L2, and the kernel's whole traffic once A is larger than
// the L2 (32,768 rows of width 5,120 are 335 MB: 136 columns of tiles would read 45 GB).  So
// the rows of tiles are taken in groups of `group_m` whose slice of A fits the L2: within a
// group down the rows, then the next column, and only then the next group.  Every tile is
// still computed once, by one CTA (or pair), over the whole of K: the result is the same.
__device__ __forceinline__ void tile_of(int t, int tiles_m, int tiles_n, int group_m, int &tm, int &tn) {
  const int per_group = group_m * tiles_n;
  const int grp = t / per_group, within = t - grp * per_group;
  const int rows = min(group_m, tiles_m - grp * group_m);       // the last group may be shorter
  tn = within / rows;
  tm = grp * group_m + (within - tn * rows);
}

// ---- persistent variant -----------------------------------------------------------------
// One CTA per SM walks over tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... (tile t covers
// rows 128 * (t % tiles_m), columns BN * (t / tiles_m): the CTAs that run at the same time
// share a few panels of W and all of A in the L2).  The accumulator is double-buffered in
// tensor memory (2 x BN columns): while the epilogue warps drain tile j, the MMAs of tile j+1
// run, and the producer's ring of stages never drains between tiles.  Same roles, same bounded
// waits and status codes as above.
#ifdef G2B_GEMM_TIMING
// Development aid (off unless built with -DG2B_GEMM_TIMING): cycles that the roles of CTA 0
// spend waiting and working, read back with g2b_gemm_tc_timing.
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

template <int BN, int STAGES> struct SmemP {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SCRATCH_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int SCRATCH_BYTES = 4 * 2 * 4096;          // two 32 x 128-byte boxes per epilogue warp
  static constexpr int BARRIER_OFFSET = SCRATCH_OFFSET + SCRATCH_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BARRIER_OFFSET + 8 * (2 * STAGES + 5) + 16 + 1024;   // + barriers, slot, alignment slack
};

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                          const __grid_constant__ CUtensorMap map_c, int M, int N, int K, int group_m,
                          int k_parts, int *__restrict__ status) {
  pdl_launch();
  extern __shared__ unsigned char smem_raw[];
  using S = SmemP<BN, STAGES>;
  unsigned char *smem = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + S::BARRIER_OFFSET);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 5);
  const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + STAGES);
  const uint32_t acc_full0 = smem_addr(bars + 2 * STAGES), acc_empty0 = smem_addr(bars + 2 * STAGES + 2);
  const uint32_t part_bar = smem_addr(bars + 2 * STAGES + 4);     // the other ranks' parts of my chunks

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = (K + BK - 1) / BK;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  // K in parts (k_parts > 1): a cluster per tile, one tile per cluster (the host sees to it),
  // rank r takes the blocks [r nkb / k_parts, (r + 1) nkb / k_parts) of K
  const int rank = k_parts > 1 ? (int)cluster_ctarank() : 0;
  const int walker = (int)blockIdx.x / k_parts, walkers = (int)gridDim.x / k_parts;
  const int n_tiles = k_parts > 1 ? min(tiles_m * tiles_n, walkers) : tiles_m * tiles_n;
  const int kb_lo = (int)((long long)nkb * rank / k_parts), kb_hi = (int)((long long)nkb * (rank + 1) / k_parts);
  const int n_kb = kb_hi - kb_lo;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 4);            // one arrival per epilogue warp
    }
    mbar_init(part_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    if (k_parts > 1) {
      const int own = part_chunk_lo<BN, EPI>(rank + 1, k_parts) - part_chunk_lo<BN, EPI>(rank, k_parts);
      if (walker < n_tiles && own > 0) mbar_expect_tx(part_bar, (uint32_t)((k_parts - 1) * own) * PART_CHUNK_BYTES);
    }
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                     smem_addr(tmem_slot)), "r"((uint32_t)(2 * BN)));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  // the weights of the first ring (this CTA's first tile) are requested above the dependency
  // line: they do not depend on the kernels in front; the rows of A follow below it
  const int n_early = walker < n_tiles ? min(n_kb, STAGES) : 0;
  if (warp == 4 && lane == 0 && PRODUCER_RUNS) {
    int tm, tn;
    tile_of(walker, tiles_m, tiles_n, group_m, tm, tn);
    const int n0 = tn * BN;
    for (int kb = 0; kb < n_early; ++kb) {
      mbar_expect_tx(full0 + 8 * kb, S::STAGE_BYTES);
      tma_load_2d(smem_addr(smem + kb * S::STAGE_BYTES) + S::A_BYTES, &map_w, (kb_lo + kb) * BK, n0, full0 + 8 * kb);
    }
  }
  pdl_wait();

  if (warp == 4) {
    if (lane == 0 && PRODUCER_RUNS) {
      uint32_t g = 0;                                // k-blocks loaded so far, over all tiles
      bool ok = true;
      TDECL(0); TDECL(1);
      TICK(t_prod);
      for (int t = walker; t < n_tiles && ok; t += walkers) {
        int tm, tn;
        tile_of(t, tiles_m, tiles_n, group_m, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++g) {
          const uint32_t s = g % STAGES;
          TICK(t_e);
          if (g >= STAGES && !mbar_wait(empty0 + 8 * s, ((g / STAGES) - 1) & 1)) {
            atomicExch(status, ST_PRODUCER_TIMEOUT);
            ok = false;
            break;
          }
          TOCK(1, t_e);
          const uint32_t a_dst = smem_addr(smem + s * S::STAGE_BYTES);
          if ((int)g >= n_early) {                           // the first ring's weights are on their way
            mbar_expect_tx(full0 + 8 * s, S::STAGE_BYTES);
            tma_load_2d(a_dst + S::A_BYTES, &map_w, kb * BK, n0, full0 + 8 * s);
          }
          tma_load_2d(a_dst, &map_a, kb * BK, m0, full0 + 8 * s);
        }
      }
      TOCK(0, t_prod);
      TFLUSH(0); TFLUSH(1);
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_n(BN);
      uint32_t g = 0, j = 0;                         // k-blocks and tiles so far
      bool ok = true;
      TDECL(2); TDECL(3); TDECL(4); TDECL(5);
      TICK(t_mma);
      for (int t = walker; t < n_tiles && ok; t += walkers, ++j) {
        const uint32_t buf = j & 1;
        // the epilogue must have drained this accumulator (it was used by tile j - 2)
        TICK(t_ae);
        if (j >= 2 && !mbar_wait(acc_empty0 + 8 * buf, ((j >> 1) - 1) & 1)) {
          atomicExch(status, ST_MMA_TIMEOUT);
          break;
        }
        TOCK(3, t_ae);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        for (int kb = 0; kb < n_kb; ++kb, ++g) {
          const uint32_t s = g % STAGES;
          TICK(t_f);
          if (!mbar_wait(full0 + 8 * s, (g / STAGES) & 1)) {
            atomicExch(status, ST_MMA_TIMEOUT);
            ok = false;
            break;
          }
          TOCK(4, t_f);
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t a_addr = smem_addr(smem + s * S::STAGE_BYTES);
          const uint64_t adesc = desc_k_major(a_addr), bdesc = desc_k_major(a_addr + S::A_BYTES);
          TICK(t_i);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16(tmem + buf * BN, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(empty0 + 8 * s);
          TOCK(5, t_i);
        }
        if (ok) umma_commit(acc_full0 + 8 * buf);    // this tile's MMAs have completed
      }
      TOCK(2, t_mma);
      TFLUSH(2); TFLUSH(3); TFLUSH(4); TFLUSH(5);
    }
  } else if (k_parts == 1) {
    unsigned char *stage = smem + S::SCRATCH_OFFSET + warp * (2 * 4096);
    uint32_t j = 0, box = 0;
    TDECL(6); TDECL(7); TDECL(8);
    TICK(t_epi);
    for (int t = walker; t < n_tiles; t += walkers, ++j) {
      const uint32_t buf = j & 1;
      TICK(t_af);
      if (!mbar_wait(acc_full0 + 8 * buf, (j >> 1) & 1)) {
        if (lane == 0) atomicExch(status, ST_EPILOGUE_TIMEOUT);
        break;
      }
      TOCK(7, t_af);
      TOCK(8, t_af - 1 + clock64());               // counts tiles (adds 1)
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      int tm, tn;
      tile_of(t, tiles_m, tiles_n, group_m, tm, tn);
      const int m0 = tm * BM, n0 = tn * BN;
      epilogue_tile_bulk<BN, EPI>(tmem + buf * BN, stage, &map_c, m0, n0, M, N, warp, lane, box);
      // every load of this warp from the accumulator has completed (each is waited for)
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
    }
    if (lane == 0) bulk_wait<0>();                 // the staging buffers are read and C is written
    TOCK(6, t_epi);
    if (threadIdx.x == 0) { TFLUSH(6); TFLUSH(7); TFLUSH(8); }
  }
  if (k_parts > 1) {
    // every thread of every CTA of the cluster comes through here, whatever its waits did
    const bool have_tile = walker < n_tiles;
    bool have_acc = false;
    if (warp < 4 && have_tile) {
      have_acc = mbar_wait(acc_full0, 0);            // this rank's products are complete: its ring is free
      if (!have_acc && lane == 0) atomicExch(status, ST_EPILOGUE_TIMEOUT);
      have_acc = __all_sync(0xffffffffu, have_acc);
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      if (have_acc) parts_lay_out<BN, EPI>(tmem, smem, warp, lane, rank, k_parts);
      fence_async_shared();                          // the bulk copies below read what was just written
    }
    cluster_sync_all();                              // every rank's ring is free and its chunks for the others lie ready
    if (warp < 4 && have_tile) {
      if (threadIdx.x == 0 && have_acc) parts_send<BN, EPI>(smem, part_bar, rank, k_parts);
      const int own = part_chunk_lo<BN, EPI>(rank + 1, k_parts) - part_chunk_lo<BN, EPI>(rank, k_parts);
      if (have_acc && own > 0) {
        have_acc = mbar_wait(part_bar, 0);           // the other ranks' parts of my chunks have arrived
        if (!have_acc && lane == 0) atomicExch(status, ST_EPILOGUE_TIMEOUT);
        have_acc = __all_sync(0xffffffffu, have_acc);
      }
      if (have_acc && own > 0) {
        unsigned char *stage = smem + S::SCRATCH_OFFSET + warp * (2 * 4096);
        uint32_t box = 0;
        int tm, tn;
        tile_of(walker, tiles_m, tiles_n, group_m, tm, tn);
        parts_finish<BN, EPI>(tmem, smem, stage, &map_c, tm * BM, tn * BN, M, N, warp, lane, box, rank, k_parts);
      }
      if (lane == 0) bulk_wait<0>();
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"((uint32_t)(2 * BN)));
  }
  // the copies that read this CTA's ring and the arrivals on its barrier are over when every
  // rank has its parts: nobody leaves before
  if (k_parts > 1) cluster_sync_all();
}

// ---- pairs of CTAs -------------------------------------------------------------------------
// A cluster of two CTAs (on two SMs) computes a 256 x BN tile of C with tcgen05.mma
// cta_group::2: each CTA brings its own 128 rows of A and half of the BN rows of W (the even
// CTA, the leader, the first half), so for BN = 256 a CTA takes in 32 KB for every 64-wide
// block of K instead of the 48 KB of a 128 x 256 tile by itself, and the ring is six blocks deep.  One
// thread of the leader issues the products for both; the accumulator of a CTA is its own 128
// rows x BN columns of tensor memory (two of them, as above), and each CTA's epilogue warps
// write its rows.  Barriers: "full" lives in the leader and counts the bytes of both CTAs'
// copies; "empty" and "accumulator ready" exist in both and are signalled in both by one
// commit; "accumulator drained" lives in the leader and gets the arrivals of all eight
// epilogue warps.  Pairs walk over tiles t = pair, pair + pairs, ...  Before it frees its
// tensor memory and exits, a CTA tells its peer that it is done and waits for the same from
// it (bounded like every other wait): the peer's products read this CTA's shared memory and
// write its tensor memory, and its barriers get arrivals from there.
template <int BN, int STAGES> struct SmemPair {
  static constexpr int A_BYTES = BM * BK * 2;                 // this CTA's 128 rows of A
  static constexpr int B_BYTES = (BN / 2) * BK * 2;           // this CTA's half of the tile's rows of W
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SCRATCH_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int SCRATCH_BYTES = 4 * 2 * 4096;          // two 32 x 128-byte boxes per epilogue warp
  static constexpr int BARRIER_OFFSET = SCRATCH_OFFSET + SCRATCH_BYTES;
  static constexpr int N_BARRIERS = 2 * STAGES + 5;           // full, empty, 2 ready, 2 drained, done
  static constexpr int TOTAL = BARRIER_OFFSET + 8 * N_BARRIERS + 16 + 1024;   // + slot, alignment slack
};

enum { ST_PAIR_TIMEOUT = 4 };

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_c, int M, int N, int K, int group_m,
                    int *__restrict__ status) {
  pdl_launch();
  extern __shared__ unsigned char smem_raw[];
  using S = SmemPair<BN, STAGES>;
  unsigned char *smem = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + S::BARRIER_OFFSET);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + S::N_BARRIERS);
  const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + STAGES);
  const uint32_t acc_full0 = smem_addr(bars + 2 * STAGES), acc_empty0 = smem_addr(bars + 2 * STAGES + 2);
  const uint32_t done_bar = smem_addr(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();               // 0: the leader
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int nkb = (K + BK - 1) / BK;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);                   // the leader's producer, with both CTAs' bytes
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 8);            // one arrival per epilogue warp of both CTAs
    }
    mbar_init(done_bar, 1);
    mbar_init_fence();
  }
  if (warp == 5) tmem_alloc_pair(smem_addr(tmem_slot), (uint32_t)(2 * BN));
  tc_fence_before();
  cluster_sync_all();                              // both CTAs' barriers and tensor memory exist
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();

  if (warp == 4) {
    if (lane == 0 && PRODUCER_RUNS) {
      const uint32_t leader_full0 = map_to_cta(full0, 0);
      uint32_t g = 0;                                // k-blocks loaded so far, over all tiles
      bool ok = true;
      for (int t = pair; t < n_tiles && ok; t += pairs) {
        int tm, tn;
        tile_of(t, tiles_m, tiles_n, group_m, tm, tn);
        const int m0 = tm * (2 * BM) + (int)rank * BM;
        const int n0 = tn * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < nkb; ++kb, ++g) {
          const uint32_t s = g % STAGES;
          if (g >= STAGES && !mbar_wait(empty0 + 8 * s, ((g / STAGES) - 1) & 1)) {
            atomicExch(status, ST_PRODUCER_TIMEOUT);
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_addr(smem + s * S::STAGE_BYTES);
          if (leader) mbar_expect_tx(full0 + 8 * s, 2 * S::STAGE_BYTES);
          tma_load_2d_pair(a_dst, &map_a, kb * BK, m0, leader_full0 + 8 * s);
          tma_load_2d_pair(a_dst + S::A_BYTES, &map_w, kb * BK, n0, leader_full0 + 8 * s);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = instr_desc(2 * BM, BN, false);
      uint32_t g = 0, j = 0;                         // k-blocks and tiles so far
      bool ok = true;
      for (int t = pair; t < n_tiles && ok; t += pairs, ++j) {
        const uint32_t buf = j & 1;
        // both CTAs' epilogues must have drained this accumulator (it was used by tile j - 2)
        if (j >= 2 && !mbar_wait(acc_empty0 + 8 * buf, ((j >> 1) - 1) & 1)) {
          atomicExch(status, ST_MMA_TIMEOUT);
          break;
        }
        tc_fence_after();
        for (int kb = 0; kb < nkb; ++kb, ++g) {
          const uint32_t s = g % STAGES;
          if (!mbar_wait(full0 + 8 * s, (g / STAGES) & 1)) {
            atomicExch(status, ST_MMA_TIMEOUT);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_addr(smem + s * S::STAGE_BYTES);
          const uint64_t adesc = desc_k_major(a_addr), bdesc = desc_k_major(a_addr + S::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16_pair(tmem + buf * BN, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(empty0 + 8 * s, 3);       // the stage is free in both CTAs
        }
        if (ok) umma_commit_pair(acc_full0 + 8 * buf, 3);   // this tile's products have completed
      }
    }
  } else {
    unsigned char *stage = smem + S::SCRATCH_OFFSET + warp * (2 * 4096);
    const uint32_t leader_acc_empty0 = map_to_cta(acc_empty0, 0);
    uint32_t j = 0, box = 0;
    for (int t = pair; t < n_tiles; t += pairs, ++j) {
      const uint32_t buf = j & 1;
      if (!mbar_wait(acc_full0 + 8 * buf, (j >> 1) & 1)) {
        if (lane == 0) atomicExch(status, ST_EPILOGUE_TIMEOUT);
        break;
      }
      tc_fence_after();
      int tm, tn;
      tile_of(t, tiles_m, tiles_n, group_m, tm, tn);
      const int m0 = tm * (2 * BM) + (int)rank * BM, n0 = tn * BN;
      epilogue_tile_bulk<BN, EPI>(tmem + buf * BN, stage, &map_c, m0, n0, M, N, warp, lane, box);
      // every load of this warp from the accumulator has completed (each is waited for)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_acc_empty0 + 8 * buf);
    }
    if (lane == 0) bulk_wait<0>();                 // the staging buffers are read and C is written
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    // this CTA issues and receives nothing more: tell the peer, and wait for the same from it
    if (lane == 0) {
      mbar_arrive_cluster(map_to_cta(done_bar, rank ^ 1u));
      if (!mbar_wait(done_bar, 0)) atomicExch(status, ST_PAIR_TIMEOUT);
    }
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem, (uint32_t)(2 * BN));
  }
}

// ---- weight streaming for 17 to 128 rows -------------------------------------------------------
// With so few rows the time goes to reading W once, and a 128 x 64 tile of C per CTA leaves the
// memory idle: N / 64 CTAs, each with a ring that is two thirds rows of A.  Here the operands are
// swapped: a CTA owns 128 rows of W (the 128-row operand of the product, 16 KB per block of K) and
// all rows of A (the narrow operand: BNB = 32, 64 or 128 of them), so that a stage is mostly
// weights; and a cluster of S CTAs shares a tile, each taking a contiguous part of K.  Their
// partial tiles are added in rank order, by all of them: after a cluster barrier (every CTA's
// products are done, so the rings are free) each CTA lays its accumulator out in its own shared
// memory; the rows of A are dealt out to the CTAs in equal ranges, and a CTA sends every other
// one that one's range of its tile with a bulk copy through the cluster's window; a CTA waits
// for the bytes it is due, a second cluster barrier tells everybody that all copies have
// arrived, and each CTA adds the S tiles of its range in rank order and writes those rows of C.
// The accumulator holds C transposed (lane = row of W, column = row of A); on the way through
// shared memory it is turned, so that C is written in rows, four outputs per lane.
// Every wait on an mbarrier is bounded as above and no role leaves before the two cluster
// barriers, whatever it has recorded in `status`.
template <int BNB, int STAGES> struct SmemWS {
  static constexpr int W_BYTES = BM * BK * 2;
  static constexpr int A_BYTES = BNB * BK * 2;
  static constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BARRIER_OFFSET = RING_BYTES;
  static constexpr int TOTAL = BARRIER_OFFSET + 8 * (2 * STAGES + 3) + 1024;   // + slot, one more barrier, alignment slack
};

template <int BNB, int STAGES, int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_tc_wstream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                       void *__restrict__ Cv, int M, int N, int K, int ldc, int splits,
                       int *__restrict__ status) {
  pdl_launch();
  extern __shared__ unsigned char smem_raw[];
  using S = SmemWS<BNB, STAGES>;
  unsigned char *smem = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + S::BARRIER_OFFSET);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 1);
  const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + STAGES);
  const uint32_t acc_bar = smem_addr(bars + 2 * STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)(blockIdx.x % (unsigned)splits);        // = the CTA's rank in its cluster
  const int n0 = (int)(blockIdx.x / (unsigned)splits) * BM;
  const int nkb = (K + BK - 1) / BK;
  const int per = (nkb + splits - 1) / splits;
  const int kb_lo = rank * per, kb_hi = min(nkb, kb_lo + per);   // this CTA's blocks of K (never empty)
  // CTAs that run side by side would all read the same columns of rows that lie a power of two
  // apart, which lands on few memory channels: every tile starts its walk over K somewhere else
  // (and wraps around), so that the order of its sum depends on the tile only
  const int n_loc = kb_hi - kb_lo;
  const int rot = (int)((blockIdx.x / (unsigned)splits) * 5u % (unsigned)n_loc);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(acc_bar, 1);
    mbar_init_fence();
  }
  if (warp == 5) tmem_alloc(smem_addr(tmem_slot), (uint32_t)BNB);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // The weights do not depend on the kernels in front: the first ring of them is requested
  // above the dependency line (a stage's barrier expects the stage's whole byte count; the
  // rows of A follow below the line).
  const int n_early = min(n_loc, STAGES);
  if (warp == 4 && lane == 0 && PRODUCER_RUNS) {
    for (int i = 0; i < n_early; ++i) {
      const int kb = kb_lo + (i + rot) % n_loc;
      mbar_expect_tx(full0 + 8 * i, S::STAGE_BYTES);
      tma_load_2d(smem_addr(smem + i * S::STAGE_BYTES), &map_w, kb * BK, n0, full0 + 8 * i);
    }
  }
  pdl_wait();                  // barriers and tensor memory are set up; now the inputs are needed

#ifdef G2B_GEMM_TIMING
  // stamps of CTA 0 (a leader) and CTA 1 (its first peer), thread 0: after set-up, accumulator
  // complete, first cluster barrier passed, tile staged / arrived, second barrier passed, end
#define TSTAMP(i) if (threadIdx.x == 0 && blockIdx.x < 2) g2b_timing[8 * blockIdx.x + (i)] = (unsigned long long)clock64()
#else
#define TSTAMP(i)
#endif
  TSTAMP(0);
  bool have_acc = true;        // epilogue warps: the accumulator is complete
  if (warp == 4) {
    if (lane == 0 && PRODUCER_RUNS) {
      for (int i = 0; i < n_loc; ++i) {
        const int kb = kb_lo + (i + rot) % n_loc, s = i % STAGES;
        if (i >= STAGES && !mbar_wait(empty0 + 8 * s, ((i / STAGES) - 1) & 1)) {
          atomicExch(status, ST_PRODUCER_TIMEOUT);
          break;
        }
        const uint32_t w_dst = smem_addr(smem + s * S::STAGE_BYTES);
        if (i >= n_early) {                                  // the first ring's weights are on their way
          mbar_expect_tx(full0 + 8 * s, S::STAGE_BYTES);
          tma_load_2d(w_dst, &map_w, kb * BK, n0, full0 + 8 * s);
        }
        tma_load_2d(w_dst + S::W_BYTES, &map_a, kb * BK, 0, full0 + 8 * s);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(BM, BNB, false);
      for (int i = 0; i < n_loc; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(full0 + 8 * s, (i / STAGES) & 1)) {
          atomicExch(status, ST_MMA_TIMEOUT);
          break;
        }
        tc_fence_after();
        const uint32_t w_addr = smem_addr(smem + s * S::STAGE_BYTES);
        const uint64_t wdesc = desc_k_major(w_addr), adesc = desc_k_major(w_addr + S::W_BYTES);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          umma_bf16(tmem, wdesc + 2 * k, adesc + 2 * k, idesc, (i | k) != 0 ? 1u : 0u);
        umma_commit(empty0 + 8 * s);
      }
      umma_commit(acc_bar);                          // all products issued so far have completed
    }
  } else {
    if (!mbar_wait(acc_bar, 0)) {
      if (lane == 0) atomicExch(status, ST_EPILOGUE_TIMEOUT);
      have_acc = false;
    }
    have_acc = __all_sync(0xffffffffu, have_acc);    // the same for the whole warp
    tc_fence_after();
  }
  TSTAMP(1);

  // Every CTA lays its partial tile out in its own ring as [row of A][128 rows of W] floats (the 32
  // lanes of a warp write 32 consecutive floats).  With K in parts, the rows of A are dealt out to
  // the CTAs of the cluster in equal ranges: a CTA sends every other CTA that one's range of its
  // tile with one bulk copy through the cluster's window (the bytes are counted on a barrier of
  // the receiver), then adds the S tiles of its own range in rank order and writes those rows of C.
  float *tile = reinterpret_cast<float *>(smem);                                 // [BNB][128]
  float *recv = tile + (size_t)BNB * BM;                                         // [sender][rows of my range][128]
  const uint32_t part_bar = smem_addr(bars + 2 * STAGES + 1 + 1);               // after the tensor-memory slot
  const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16);
  const int nl = warp * 32 + lane;                   // this thread's row of W within the tile
  const int m_all = min(M, BNB);
  const int mq = (m_all + splits - 1) / splits;      // rows of A per CTA of the cluster
  const int m_lo = min(m_all, rank * mq), m_hi = min(m_all, m_lo + mq);          // this CTA's range
  if (splits > 1) {
    if (threadIdx.x == 0) {
      mbar_init(part_bar, 1);
      mbar_init_fence();
      mbar_expect_tx(part_bar, (uint32_t)(splits - 1) * (uint32_t)(m_hi - m_lo) * BM * 4);
    }
    tc_fence_before();
    cluster_sync_all();                              // every CTA's products are done: the rings are free
    tc_fence_after();
    TSTAMP(2);
  }
  if (warp < 4 && have_acc) {
#pragma unroll 1
    for (int c0 = 0; c0 < m_all; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(taddr + (uint32_t)c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (c0 + j < m_all) tile[(size_t)(c0 + j) * BM + nl] = __uint_as_float(r[j]);
    }
  }
  if (splits > 1) {
    fence_async_shared();                            // the bulk copies below read what was just written
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int q = 0; q < splits; ++q) {
        const int q_lo = min(m_all, q * mq), q_hi = min(m_all, q_lo + mq);
        if (q == rank || q_hi <= q_lo) continue;
        asm volatile(
            "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
            ::"r"(map_to_cta(smem_addr(recv) + (uint32_t)rank * (uint32_t)mq * BM * 4, (uint32_t)q)),
              "r"(smem_addr(tile) + (uint32_t)q_lo * BM * 4), "r"((uint32_t)(q_hi - q_lo) * BM * 4),
              "r"(map_to_cta(part_bar, (uint32_t)q))
            : "memory");
      }
    }
    if (warp < 4) {
      if (m_hi > m_lo && !mbar_wait(part_bar, 0)) {  // the other CTAs' rows of my range have arrived
        if (lane == 0) atomicExch(status, ST_EPILOGUE_TIMEOUT);
        have_acc = false;
      }
      have_acc = __all_sync(0xffffffffu, have_acc);
    }
    TSTAMP(3);
    tc_fence_before();
    cluster_sync_all();                              // every copy has arrived: nobody's tile is needed any more
    tc_fence_after();
    TSTAMP(4);
  } else {
    if (warp < 4) asm volatile("bar.sync 1, 128;\n" ::: "memory");       // the four epilogue warps
  }
  if (warp < 4 && have_acc) {
    // this CTA's rows of C: a warp takes every fourth row of A, a lane four neighbours of the
    // row's 128 outputs
    const int n = n0 + 4 * lane;
    const bool vec_ok = ((((uintptr_t)Cv) | ((size_t)ldc * 4)) & 15) == 0;
    for (int m = m_lo + warp; m < m_hi; m += 4) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        if (p < splits) {
          const float *src = p == rank ? tile + (size_t)m * BM : recv + ((size_t)p * mq + (m - m_lo)) * BM;
          const float4 t = *reinterpret_cast<const float4 *>(src + 4 * lane);
          v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
        }
      }
      if (EPI == EPI_SWIGLU_BF16) {
        // rows 16b .. 16b+7 of W are gates (lanes 4b, 4b+1), 16b+8 .. 16b+15 the ups (lanes 4b+2, 4b+3)
        float4 up;
        up.x = __shfl_down_sync(0xffffffffu, v.x, 2); up.y = __shfl_down_sync(0xffffffffu, v.y, 2);
        up.z = __shfl_down_sync(0xffffffffu, v.z, 2); up.w = __shfl_down_sync(0xffffffffu, v.w, 2);
        if ((lane & 2) == 0) {
          const int col = ((n >> 4) << 3) + (n & 7);          // output column of v.x
          bf16 *dst = (bf16 *)Cv + (size_t)m * ldc + col;
          const float h0 = __fdividef(v.x, 1.f + __expf(-v.x)) * up.x, h1 = __fdividef(v.y, 1.f + __expf(-v.y)) * up.y;
          const float h2 = __fdividef(v.z, 1.f + __expf(-v.z)) * up.z, h3 = __fdividef(v.w, 1.f + __expf(-v.w)) * up.w;
          if (n + 16 <= N && ((((uintptr_t)dst) & 7) == 0)) {
            *reinterpret_cast<uint2 *>(dst) = make_uint2(pack2f(h0, h1), pack2f(h2, h3));
          } else {
            const float h[4] = {h0, h1, h2, h3};
            for (int e = 0; e < 4; ++e)
              if (n + 8 + e < N) dst[e] = __float2bfloat16_rn(h[e]);
          }
        }
      } else {
        const size_t o = (size_t)m * ldc + n;
        const float f[4] = {v.x, v.y, v.z, v.w};
        if (EPI == EPI_STORE_BF16) {
          bf16 *dst = (bf16 *)Cv + o;
          if (n + 4 <= N && ((((uintptr_t)dst) & 7) == 0)) {
            *reinterpret_cast<uint2 *>(dst) = make_uint2(pack2f(v.x, v.y), pack2f(v.z, v.w));
          } else {
            for (int e = 0; e < 4; ++e)
              if (n + e < N) dst[e] = __float2bfloat16_rn(f[e]);
          }
        } else if (EPI == EPI_STORE_F32) {
          float *dst = (float *)Cv + o;
          if (n + 4 <= N && vec_ok) {
            *reinterpret_cast<float4 *>(dst) = v;
          } else {
            for (int e = 0; e < 4; ++e)
              if (n + e < N) dst[e] = f[e];
          }
        } else {
          float *dst = (float *)Cv + o;            // a reduction: one add per element and launch
          if (n + 4 <= N && vec_ok) {
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z),
                         "f"(v.w) : "memory");
          } else {
            for (int e = 0; e < 4; ++e)
              if (n + e < N) atomicAdd(dst + e, f[e]);
          }
        }
      }
    }
  }
  TSTAMP(5);
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, (uint32_t)BNB);
  }
}
#undef TSTAMP

// ---- host side ----------------------------------------------------------------------
// Tensor maps come from tc::get_map (kept by address and sizes).
static int make_map(CUtensorMap *map, const void *base, int rows, int K, int ld, int box_rows) {
  const int rc = get_map(map, base, rows, K, ld, box_rows);
  if (rc) G2B_REFUSE("gemm_tc: cuTensorMapEncodeTiled failed or is not available (code %d)", rc);
  return 0;
}

// A map of C for the tile stores of the persistent kernel: boxes of 32 rows x 128 bytes.
static int make_map_c(CUtensorMap *map, const void *base, int rows, int cols, int ld, bool is_float) {
  const int rc = get_map(map, base, rows, cols, ld, 32, is_float ? 4 : 2);
  if (rc) G2B_REFUSE("gemm_tc: cuTensorMapEncodeTiled for C failed or is not available (code %d)", rc);
  return 0;
}

template <int BN, int STAGES, int EPI>
static int launch(const CUtensorMap &ma, const CUtensorMap &mw, void *C, int M, int N, int K, int ldc,
                  int *status, cudaStream_t stream) {
  static G2bPerDevice configured;
  const int smem = Smem<BN, STAGES>::TOTAL;
  const int cfg_dev = g2b_current_device();
  if (cfg_dev < 0 || !configured.value[cfg_dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, EPI>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) G2B_REFUSE("gemm_tc: shared memory of %d bytes refused: %s", smem, cudaGetErrorString(e));
    if (cfg_dev >= 0) configured.value[cfg_dev] = 1;
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) G2B_REFUSE("gemm_tc: M=%d is too large for one launch", M);
  g2b_launch(gemm_tc_kernel<BN, STAGES, EPI>, dim3(grid), dim3(THREADS), smem, stream, ma, mw, C, M, N, K, ldc, status);
  return g2b_check_launch("gemm_tc");
}

static int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

// Rows of tiles per group (see tile_of): all of them while A fits the L2 with room for the
// panels of W (up to 48 MB); else as many as keep a group's slice of A near 32 MB.
static int rows_of_tiles_per_group(int tiles_m, int tile_rows, int K) {
  const long long tile_bytes = (long long)tile_rows * K * 2;
  if (tile_bytes * tiles_m <= (48ll << 20)) return tiles_m;
  const long long g = (32ll << 20) / tile_bytes;       // measured at 16 to 96 MB: 32 to 48 are the fastest
  return (int)(g < 1 ? 1 : (g > tiles_m ? tiles_m : g));
}

// Clusters of `sz` CTAs of the persistent kernel that the GPU holds at once (clusters do not
// straddle its processing clusters, so it can be fewer than SMs / sz): asked of the runtime once
// per device, tile width and size, for the kernel with the adding epilogue (the others use the
// same shared memory).
static int clusters_at_once(int bn, int sz) {
  static G2bPerDevice fit[2][5];                  // value[device] = answer + 1; 0 = not asked yet
  const int dev = g2b_current_device();
  if (sz < 2 || sz > 4) return 0;
  if (dev < 0 || !fit[bn == 256][sz].value[dev]) {
    // all six answers at the first question on a device (not one by one in the middle of a step)
    for (int w = 0; w < 2; ++w)
      for (int s = 2; s <= 4; ++s) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(s * sm_count()));
        cfg.blockDim = dim3(THREADS);
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)s;
        attr[0].val.clusterDim.y = attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        cudaError_t e;
        if (w) {
          cfg.dynamicSmemBytes = SmemP<256, 4>::TOTAL;
          cudaFuncSetAttribute(gemm_tc_persistent_kernel<256, 4, EPI_ACCUM_F32>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, SmemP<256, 4>::TOTAL);
          e = cudaOccupancyMaxActiveClusters(&n, gemm_tc_persistent_kernel<256, 4, EPI_ACCUM_F32>, &cfg);
        } else {
          cfg.dynamicSmemBytes = SmemP<128, 6>::TOTAL;
          cudaFuncSetAttribute(gemm_tc_persistent_kernel<128, 6, EPI_ACCUM_F32>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, SmemP<128, 6>::TOTAL);
          e = cudaOccupancyMaxActiveClusters(&n, gemm_tc_persistent_kernel<128, 6, EPI_ACCUM_F32>, &cfg);
        }
        if (e != cudaSuccess) {
          cudaGetLastError();
          n = sm_count() / s / 2;                  // a cautious guess
        }
        if (dev >= 0) fit[w][s].value[dev] = n + 1;
        else if (w == (bn == 256) && s == sz) return n;
      }
  }
  return fit[bn == 256][sz].value[dev] - 1;
}

// The persistent kernel's tile width (128 with six stages or 256 with four) and parts of K for
// a product, from a small model of its time in microseconds, fitted to measurements on a B200
// at 192 to 2,048 rows against the matrices of three model sizes: rounds of tiles per CTA x
// blocks of K per part x 0.295 (0.34 for the wide tile), plus what the exchange of the parts
// costs (2.3 for the narrow tile, 1.4 + 1.5 per part for the wide one).  K goes in parts only
// when all clusters run at once, a part has at least 8 blocks and the parts save at least 12.
static void choose_persistent(int M, int N, int K, int epi, int *bn_out, int *parts_out, int only_bn) {
  const int nkb = (K + BK - 1) / BK, tiles_m = (M + BM - 1) / BM, sms = sm_count();
  double best = 1e30;
  for (int w = 0; w < 2; ++w) {
    const int bn = w ? 256 : 128;
    if (only_bn && bn != only_bn) continue;
    const long long tiles = (long long)tiles_m * ((N + bn - 1) / bn);
    const double t_kb = w ? 0.34 : 0.295;
    for (int p = 1; p <= 4; ++p) {
      if (p > 1 && (nkb / p < 8 || (long long)nkb * (p - 1) / p < 12 || !parts_fit(bn, epi, p, nkb, 196608) ||
                    2 * tiles > sms || tiles > clusters_at_once(bn, p)))
        continue;
      const long long rounds = (tiles * p + sms - 1) / sms;
      const double cost = (double)rounds * ((nkb + p - 1) / p) * t_kb + (p > 1 ? (w ? 1.4 + 1.5 * p : 2.3) : 0.0);
      if (cost < best - 1e-9) {
        best = cost;
        *bn_out = bn;
        *parts_out = p;
      }
    }
  }
}
static_assert(SmemP<128, 6>::RING_BYTES == 196608 && SmemP<256, 4>::RING_BYTES == 196608, "choose_persistent's ring");

// want_parts: 1 to 4 parts of K
template <int BN, int STAGES, int EPI>
static int launch_persistent(const CUtensorMap &ma, const CUtensorMap &mw, void *C, int M, int N, int K, int ldc,
                             int want_parts, int *status, cudaStream_t stream) {
  static G2bPerDevice configured;
  const int smem = SmemP<BN, STAGES>::TOTAL;
  const int cfg_dev = g2b_current_device();
  if (cfg_dev < 0 || !configured.value[cfg_dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, STAGES, EPI>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) G2B_REFUSE("gemm_tc: shared memory of %d bytes refused: %s", smem, cudaGetErrorString(e));
    if (cfg_dev >= 0) configured.value[cfg_dev] = 1;
  }
  const long long tiles = (long long)((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  if (tiles > 0x7fffffffLL) G2B_REFUSE("gemm_tc: %lld tiles", tiles);
  const bool is_float = EPI == EPI_STORE_F32 || EPI == EPI_ACCUM_F32;
  const int c_cols = EPI == EPI_SWIGLU_BF16 ? N / 2 : N;
  if (((uintptr_t)C & 15) || (ldc * (is_float ? 4 : 2)) % 16)
    G2B_REFUSE("gemm_tc: the persistent kernel stores tiles of C: C must be 16-byte aligned with a row stride "
               "that is a multiple of 16 bytes (ldc = %d)", ldc);
  CUtensorMap mc;
  const int rc = make_map_c(&mc, C, M, c_cols, ldc, is_float);
  if (rc) return rc;
  const int nkb = (K + BK - 1) / BK;
  const int parts = want_parts < 1 ? 1 : want_parts;
  if (parts > 1) {
    if (!parts_fit(BN, EPI, parts, nkb, SmemP<BN, STAGES>::RING_BYTES))
      G2B_REFUSE("gemm_tc: %d parts of K do not fit tiles %d wide with this epilogue (K = %d)", parts, BN, K);
    const int room = clusters_at_once(BN, parts);
    if (tiles > room)
      G2B_REFUSE("gemm_tc: %lld tiles in %d parts of K are more clusters than the GPU holds at once (%d)", tiles,
                 parts, room);
  }
  const unsigned grid = parts > 1 ? (unsigned)(tiles * parts) : (unsigned)(tiles < sm_count() ? tiles : sm_count());
  g2b_launch_cluster(gemm_tc_persistent_kernel<BN, STAGES, EPI>, dim3(grid), dim3(THREADS), smem, stream,
                     (unsigned)parts, ma, mw, mc, M, N, K, rows_of_tiles_per_group((M + BM - 1) / BM, BM, K), parts,
                     status);
  return g2b_check_launch("gemm_tc (persistent)");
}

template <int BN, int STAGES, int EPI>
static int launch_pair(const CUtensorMap &ma, const CUtensorMap &mw, void *C, int M, int N, int K, int ldc,
                       int *status, cudaStream_t stream) {
  static G2bPerDevice configured;
  const int smem = SmemPair<BN, STAGES>::TOTAL;
  const int cfg_dev = g2b_current_device();
  if (cfg_dev < 0 || !configured.value[cfg_dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<BN, STAGES, EPI>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) G2B_REFUSE("gemm_tc: shared memory of %d bytes refused: %s", smem, cudaGetErrorString(e));
    if (cfg_dev >= 0) configured.value[cfg_dev] = 1;
  }
  const long long tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  if (tiles > 0x7fffffffLL) G2B_REFUSE("gemm_tc: %lld tiles", tiles);
  const bool is_float = EPI == EPI_STORE_F32 || EPI == EPI_ACCUM_F32;
  const int c_cols = EPI == EPI_SWIGLU_BF16 ? N / 2 : N;
  if (((uintptr_t)C & 15) || (ldc * (is_float ? 4 : 2)) % 16)
    G2B_REFUSE("gemm_tc: the paired kernel stores tiles of C: C must be 16-byte aligned with a row stride "
               "that is a multiple of 16 bytes (ldc = %d)", ldc);
  CUtensorMap mc;
  const int rc = make_map_c(&mc, C, M, c_cols, ldc, is_float);
  if (rc) return rc;
  const int max_pairs = sm_count() / 2;
  if (max_pairs < 1) G2B_REFUSE("gemm_tc: the paired kernel needs two SMs");
  const unsigned pairs = (unsigned)(tiles < max_pairs ? tiles : max_pairs);
  g2b_launch_cluster(gemm_tc_pair_kernel<BN, STAGES, EPI>, dim3(2 * pairs), dim3(THREADS), smem, stream, 2u, ma, mw,
                     mc, M, N, K, rows_of_tiles_per_group((M + 2 * BM - 1) / (2 * BM), 2 * BM, K), status);
  return g2b_check_launch("gemm_tc (pairs)");
}

template <int BNB, int STAGES, int EPI>
static int launch_wstream(const void *A, const void *W, void *C, int M, int N, int K, int lda, int ldw, int ldc,
                          int want_splits, int *status, cudaStream_t stream) {
  static G2bPerDevice configured;
  using S = SmemWS<BNB, STAGES>;
  const int cfg_dev = g2b_current_device();
  if (cfg_dev < 0 || !configured.value[cfg_dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_wstream_kernel<BNB, STAGES, EPI>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) G2B_REFUSE("gemm_tc: shared memory of %d bytes refused: %s", S::TOTAL, cudaGetErrorString(e));
    if (cfg_dev >= 0) configured.value[cfg_dev] = 1;
  }
  CUtensorMap mw, ma;
  int rc = make_map(&mw, W, N, K, ldw, BM);
  if (rc) return rc;
  rc = make_map(&ma, A, M, K, lda, BNB);
  if (rc) return rc;
  const int tiles = (N + BM - 1) / BM, nkb = (K + BK - 1) / BK;
  // parts of K: as many (up to 4) as keep every CTA on the GPU at once and give a part 4 blocks
  // or more; three where four would not fit (40 tiles: 120 CTAs instead of 80).  How many
  // clusters of a size the GPU holds at once is asked of the runtime: clusters do not straddle
  // the GPU's processing clusters, so it can be fewer than SMs / size.
  static G2bPerDevice fit[5];                     // fit[s].value[device] = clusters of s CTAs at once (+1; 0 = not asked yet)
  auto clusters_at_once = [&](int s) -> int {
    if (cfg_dev >= 0 && fit[s].value[cfg_dev]) return fit[s].value[cfg_dev] - 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(s * sm_count()));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = S::TOTAL;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)s;
    attr[0].val.clusterDim.y = attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_wstream_kernel<BNB, STAGES, EPI>, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = sm_count() / s / 2;                      // a cautious guess
    }
    if (cfg_dev >= 0) fit[s].value[cfg_dev] = n + 1;
    return n;
  };
  int splits = 1;
  for (int s = 2; s <= 4; ++s)
    if (nkb / s >= 4 && tiles <= clusters_at_once(s)) splits = s;
  if (want_splits >= 1 && want_splits <= 4) splits = want_splits;                           // the caller's choice
  while (splits > 1 && (splits - 1) * ((nkb + splits - 1) / splits) >= nkb) --splits;      // no empty part
  static_assert((2 * BNB + 8) * BM * 4 <= S::RING_BYTES, "the tile and the received ranges must fit the ring");
  g2b_launch_cluster(gemm_tc_wstream_kernel<BNB, STAGES, EPI>, dim3((unsigned)(tiles * splits)), dim3(THREADS),
                     S::TOTAL, stream, (unsigned)splits, mw, ma, C, M, N, K, ldc, splits, status);
  return g2b_check_launch("gemm_tc (weight streaming)");
}

// A [M,K], W [N,K] bfloat16, inner stride 1, row strides multiples of 8 elements, base
// addresses 16-byte aligned.  epi: 0 store bfloat16, 1 store float, 2 add into float,
// 3 SiLU gate (C is [M, N/2] bfloat16; N a multiple of 16).  `status` is a device int the
// kernel sets non-zero if one of its bounded waits gave up.  Tile shapes (bn, stages):
// (64,4) (64,8) (128,3) (128,6) (256,4); bn = 0 picks one from the sizes: wide tiles when
// there are plenty of them, narrow tiles with a deeper ring when the grid would not fill
// the GPU (the ring has to cover the latency of the copies by itself then).  persistent = 1:
// the variant with one CTA per SM and two accumulators, shapes (128,6) and (256,4), bn = 0 lets
// the launcher choose between them; with fewer tiles than half the SMs it takes K in parts over
// a cluster (persistent = 11 to 14 asks for 1 to 4 parts).  persistent
// = 2: pairs of CTAs on 256 x 256 tiles, shapes (256,6) and (256,4).  persistent = 3 (at most
// 128 rows; stages is ignored, bn = 1 to 4 asks for that many parts of K, anything else lets
// the launcher choose): the weight-streaming kernel with K split over a cluster.
extern "C" int g2b_gemm_tc(const void *A, const void *W, void *C, int M, int N, int K, int lda,
                           int ldw, int ldc, int epi, int bn, int stages, int persistent, int *status,
                           cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || lda % 8 || ldw % 8)
    G2B_REFUSE("gemm_tc: K=%d and the row strides (%d, %d) must be multiples of 8", K, lda, ldw);
  if (((uintptr_t)A | (uintptr_t)W) & 15) G2B_REFUSE("gemm_tc: operands must be 16-byte aligned");
  if (epi == EPI_SWIGLU_BF16 && N % 16) G2B_REFUSE("gemm_tc: gated output needs N %% 16 == 0, N=%d", N);
  if (!status) G2B_REFUSE("gemm_tc: no status word");
  if (bn == 0 && persistent != 1 && persistent < 11) {
    const long long tiles128 = (long long)((M + BM - 1) / BM) * ((N + 127) / 128);
    if (tiles128 >= 2 * 148) { bn = 128; stages = 3; }
    else { bn = 64; stages = 4; }
  }
  if (persistent == 3) {                           // 17 to 128 rows: the weights stream, K split over a cluster
    if (M > 128) G2B_REFUSE("gemm_tc: the weight-streaming kernel takes at most 128 rows, got %d", M);
    const bool crowded = (N + BM - 1) / BM > sm_count() && (bn < 1 || bn > 4);
#define G2B_CASE(E) \
    if (epi == E) {                                                                                        \
      /* more tiles than SMs (K is not split then): half the ring, so that two CTAs share an SM and */ \
      /* the tiles of the second round stream beside those of the first instead of after them       */ \
      if (M <= 32 && crowded) return launch_wstream<32, 4, E>(A, W, C, M, N, K, lda, ldw, ldc, bn, status, stream); \
      if (M <= 32) return launch_wstream<32, 9, E>(A, W, C, M, N, K, lda, ldw, ldc, bn, status, stream);   \
      if (M <= 64 && crowded) return launch_wstream<64, 4, E>(A, W, C, M, N, K, lda, ldw, ldc, bn, status, stream); \
      if (M <= 64) return launch_wstream<64, 8, E>(A, W, C, M, N, K, lda, ldw, ldc, bn, status, stream);   \
      return launch_wstream<128, 6, E>(A, W, C, M, N, K, lda, ldw, ldc, bn, status, stream);               \
    }
    G2B_CASE(EPI_STORE_BF16) G2B_CASE(EPI_STORE_F32) G2B_CASE(EPI_ACCUM_F32) G2B_CASE(EPI_SWIGLU_BF16)
#undef G2B_CASE
    G2B_REFUSE("gemm_tc: unknown epilogue %d", epi);
  }
  int parts = 1;
  if (persistent == 1 || persistent >= 11) {
    // tile width 0: the launcher chooses width and parts of K; a given width: the parts only
    // (persistent = 11 to 14: the caller's 1 to 4 parts)
    int w = bn, p = 1;
    if (bn != 0 && bn != 128 && bn != 256) G2B_REFUSE("gemm_tc: no persistent kernel for tile width %d", bn);
    if (persistent == 1 || bn == 0) choose_persistent(M, N, K, epi, &w, &p, bn);
    if (persistent >= 11) p = persistent - 10;
    if (bn == 0) { bn = w; stages = w == 256 ? 4 : 6; }
    parts = p;
  }
  CUtensorMap ma, mw;
  int rc = make_map(&ma, A, M, K, lda, BM);
  if (rc) return rc;
  if (persistent == 2) {                           // pairs of CTAs: 256 x bn tiles, bn / 2 rows of W per CTA
    if (bn != 256) G2B_REFUSE("gemm_tc: the paired kernel has tiles 256 wide, not %d", bn);
    rc = make_map(&mw, W, N, K, ldw, bn / 2);
    if (rc) return rc;
#define G2B_CASE(BN_, ST_, E) \
    if (bn == BN_ && stages == ST_ && epi == E)                                                      \
      return launch_pair<BN_, ST_, E>(ma, mw, C, M, N, K, ldc, status, stream);
#define G2B_SHAPE(BN_, ST_) \
    G2B_CASE(BN_, ST_, EPI_STORE_BF16) G2B_CASE(BN_, ST_, EPI_STORE_F32) G2B_CASE(BN_, ST_, EPI_ACCUM_F32) \
    G2B_CASE(BN_, ST_, EPI_SWIGLU_BF16)
    G2B_SHAPE(256, 6) G2B_SHAPE(256, 4)
#undef G2B_SHAPE
#undef G2B_CASE
    G2B_REFUSE("gemm_tc: no paired kernel for tile width %d with %d stages and epilogue %d", bn, stages, epi);
  }
  rc = make_map(&mw, W, N, K, ldw, bn);
  if (rc) return rc;
#define G2B_CASE(BN_, ST_, E) \
  if (persistent && bn == BN_ && stages == ST_ && epi == E)                                        \
    return launch_persistent<BN_, ST_, E>(ma, mw, C, M, N, K, ldc, parts, status, stream);
#define G2B_SHAPE(BN_, ST_) \
  G2B_CASE(BN_, ST_, EPI_STORE_BF16) G2B_CASE(BN_, ST_, EPI_STORE_F32) \
  G2B_CASE(BN_, ST_, EPI_ACCUM_F32) G2B_CASE(BN_, ST_, EPI_SWIGLU_BF16)
  G2B_SHAPE(128, 6) G2B_SHAPE(256, 4)
#undef G2B_SHAPE
#undef G2B_CASE
  if (persistent)
    G2B_REFUSE("gemm_tc: no persistent kernel for tile width %d with %d stages and epilogue %d", bn, stages, epi);
#define G2B_CASE(BN_, ST_, E) \
  if (bn == BN_ && stages == ST_ && epi == E) return launch<BN_, ST_, E>(ma, mw, C, M, N, K, ldc, status, stream);
#define G2B_SHAPE(BN_, ST_) \
  G2B_CASE(BN_, ST_, EPI_STORE_BF16) G2B_CASE(BN_, ST_, EPI_STORE_F32) \
  G2B_CASE(BN_, ST_, EPI_ACCUM_F32) G2B_CASE(BN_, ST_, EPI_SWIGLU_BF16)
  G2B_SHAPE(64, 4) G2B_SHAPE(64, 8) G2B_SHAPE(128, 3) G2B_SHAPE(128, 6) G2B_SHAPE(256, 4)
#undef G2B_SHAPE
#undef G2B_CASE
  G2B_REFUSE("gemm_tc: no kernel for tile width %d with %d stages and epilogue %d", bn, stages, epi);
}

#ifdef G2B_GEMM_TIMING
// Copies the 16 counters to `out` and clears them.
extern "C" int g2b_gemm_tc_timing(unsigned long long *out) {
  static unsigned long long zero[16] = {0};
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out, g2b_timing, sizeof(zero));
  cudaMemcpyToSymbol(g2b_timing, zero, sizeof(zero));
  return 0;
}
#endif
