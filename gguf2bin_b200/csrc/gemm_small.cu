// Matrix product for few rows (decode): C[M,N] = A[M,K] * W[N,K]^T, bfloat16 in, 32-bit
// accumulation, M <= 64.  The time goes to reading W once, so the kernel is built around
// the weight stream:
//
//  * Operands are swapped: 16 rows of W are the 16-row operand of mma.m16n8k16 and the
//    batch is the 8-wide one, so no tensor-core work is wasted on padding M to 64 or 128.
//  * A CTA owns 16 rows of W over the whole K; its 8 warps split every 256-wide block of
//    K into 32-wide pieces.  A thread loads 16 contiguous bytes (8 values of k) of rows g
//    and g+8 straight from global memory into registers.  The eight values feed two MMAs
//    under a permutation of k that is applied to both operands alike, so no shuffle and
//    no shared-memory staging of W is needed; several blocks of K are in flight at once.
//  * The activations of a K block (M x 256) are staged in shared memory (double buffer).
//  * The 8 partial sums of an output are added in warp order through shared memory: the
//    order of the sum depends on K only, not on M or on the batch's contents.
//
// Two ways of staging the activations.  `gemm_small_kernel` stages one 256-wide block of K
// at a time (any K, M up to 64).  `gemm_small_whole_kernel` stages all of A once, when
// M x K fits shared memory: its K loop then has no barrier at all and up to 8 blocks of W are
// in flight per thread.  (A variant that applied the block's RMSNorm while staging the float
// stream was measured against the norm as a kernel of its own and lost: every 16-row tile
// repeats the norm of all rows.)
//
// Epilogues: store (bfloat16 or float), add into a float matrix (the residual stream), or
// the SiLU gate on a fused gate/up matrix whose rows alternate 8 gates / 8 ups:
// out[m, 8b + r] = silu(row r of block b) * (row 8 + r)   (src/l3_math.c:57-62,
// src/l5_model.c:594-595 of AnonymoDGH/gguf2bin).
#include "common.cuh"
#include "mma.cuh"

#include <cooperative_groups.h>

G2B_DEFINE_LAST_ERROR

constexpr int WARPS = 8;
constexpr int KB = 256;                 // K block: 8 warps x 32
constexpr int XPAD = 32;                // elements of padding per staged row (64 bytes)
constexpr int XROW = KB + XPAD;
constexpr int DEPTH = 4;                // K blocks of W in flight per thread

enum { EPI_STORE_BF16 = 0, EPI_STORE_F32 = 1, EPI_ACCUM_F32 = 2, EPI_SWIGLU_BF16 = 3 };

__device__ __forceinline__ uint4 ld_stream(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

template <int MT, int EPI>
__global__ void __launch_bounds__(WARPS * 32)
gemm_small_kernel(const bf16 *__restrict__ A, const bf16 *__restrict__ W, void *__restrict__ Cv,
                  int M, int N, int K, int lda, int ldw, int ldc) {
  pdl_launch();
  constexpr int MROWS = MT * 8;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16 *xs = reinterpret_cast<bf16 *>(smem_raw);          // [2][MROWS][XROW]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int nkb = (K + KB - 1) / KB;

  const bf16 *w0 = W + (size_t)min(n0 + g, N - 1) * ldw;
  const bf16 *w1 = W + (size_t)min(n0 + g + 8, N - 1) * ldw;
  const int kw = 32 * warp + 8 * c;                       // this thread's k offset in a block

  auto load_w = [&](uint4 (&dst)[2], int kb) {
    const int k = kb * KB + kw;
    if (k < K) {
      dst[0] = ld_stream(w0 + k);
      dst[1] = ld_stream(w1 + k);
    } else {
      dst[0] = dst[1] = make_uint4(0, 0, 0, 0);
    }
  };
  auto stage_x = [&](int kb, int buf) {
    bf16 *dst = xs + (size_t)buf * MROWS * XROW;
    for (int i = threadIdx.x; i < MROWS * (KB / 8); i += WARPS * 32) {
      const int r = i / (KB / 8), piece = i % (KB / 8);
      const int k = kb * KB + piece * 8;
      bf16 *d = dst + r * XROW + piece * 8;
      if (r < M && k < K) cp_async_16(smem_u32(d), A + (size_t)r * lda + k);
      else *reinterpret_cast<uint4 *>(d) = make_uint4(0, 0, 0, 0);
    }
  };

  uint4 wb[DEPTH][2];
#pragma unroll
  for (int d = 0; d < DEPTH; ++d)
    if (d < nkb) load_w(wb[d], d);
  pdl_wait();                            // the activations come from the kernel before
  stage_x(0, 0);
  cp_async_commit();

  float acc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;

  for (int kb0 = 0; kb0 < nkb; kb0 += DEPTH) {
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      const int kb = kb0 + d;
      if (kb < nkb) {
        if (kb + 1 < nkb) stage_x(kb + 1, (kb + 1) & 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16 *xb = xs + (size_t)(kb & 1) * MROWS * XROW + 32 * warp + 8 * c;
        const uint4 a_lo = wb[d][0], a_hi = wb[d][1];
        const uint32_t a1[4] = {a_lo.x, a_hi.x, a_lo.y, a_hi.y};
        const uint32_t a2[4] = {a_lo.z, a_hi.z, a_lo.w, a_hi.w};
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint4 xv = *reinterpret_cast<const uint4 *>(xb + (size_t)(8 * mt + g) * XROW);
          mma_bf16_16816(acc[mt], a1, xv.x, xv.y);
          mma_bf16_16816(acc[mt], a2, xv.z, xv.w);
        }
        if (kb + DEPTH < nkb) load_w(wb[d], kb + DEPTH);
        __syncthreads();                 // the staged block may be overwritten two blocks on
      }
    }
  }
  cp_async_wait<0>();

  // partial sums of the 8 warps -> shared memory [warp][16 rows][MROWS], summed in warp order
  float *red = reinterpret_cast<float *>(smem_raw);
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    float *r0 = red + ((size_t)warp * 16 + g) * MROWS + 8 * mt + 2 * c;
    float *r1 = r0 + 8 * MROWS;
    r0[0] = acc[mt][0]; r0[1] = acc[mt][1];
    r1[0] = acc[mt][2]; r1[1] = acc[mt][3];
  }
  __syncthreads();
  if (EPI == EPI_SWIGLU_BF16) {
    // rows 0..7 of the tile are gates, rows 8..15 the ups of the same outputs
    for (int i = threadIdx.x; i < 8 * MROWS; i += WARPS * 32) {
      const int m = i / 8, r = i % 8;
      float gate = 0.f, up = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        gate += red[((size_t)w * 16 + r) * MROWS + m];
        up += red[((size_t)w * 16 + 8 + r) * MROWS + m];
      }
      const int col = (n0 >> 1) + r;
      if (m < M && n0 + 8 + r < N)
        ((bf16 *)Cv)[(size_t)m * ldc + col] = __float2bfloat16_rn((gate / (1.f + expf(-gate))) * up);
    }
  } else {
    for (int i = threadIdx.x; i < 16 * MROWS; i += WARPS * 32) {
      const int m = i / 16, r = i % 16;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) v += red[((size_t)w * 16 + r) * MROWS + m];
      const int n = n0 + r;
      if (m < M && n < N) {
        const size_t o = (size_t)m * ldc + n;
        if (EPI == EPI_STORE_BF16) ((bf16 *)Cv)[o] = __float2bfloat16_rn(v);
        else if (EPI == EPI_STORE_F32) ((float *)Cv)[o] = v;
        else atomicAdd((float *)Cv + o, v);   // a reduction: one add per element and launch, no load on the path
      }
    }
  }
}


// K blocks of W in flight per thread (whole-A kernel): 4 when a CTA has at most four blocks of
// K, else 8; the shallower ring frees registers, so that three blocks instead of two fit an SM.
//
// SPLIT > 1: a thread-block cluster of SPLIT CTAs shares one 16-row tile of W, each taking a
// contiguous slice of K (its part of the activations and of the weights); the CTAs leave
// their partial tiles in their own shared memory and the first CTA of the cluster adds them
// in rank order through distributed shared memory.  Narrow outputs (N = 1024 means only 64
// tiles) fill the GPU this way, and the order of the sum still depends on K and N only.
//
// NORMED: A is not bfloat16 activations but the float residual stream, and the product is that
// of its RMS-normalised rows, norm(x) . W^T with norm(x) = x / sqrt(mean(x^2) + eps) (the norm's
// per-channel weight was multiplied into W's columns when the weights were bound).  The row's
// factor is a scalar, so it is applied to the accumulators: while a warp stages a row (rounded
// to bfloat16 for the tensor cores) it sums the squares of the float values; the epilogue
// multiplies each output by its row's 1 / sqrt(sum / K + eps).  Against a norm kernel of its own
// this repeats the sum in every CTA (a few thousand additions, from the L2) but neither
// normalises nor stores anything twice, and the step has one dependent launch less.
template <int MT, int EPI, int DEPTH_WHOLE, int SPLIT, bool NORMED = false>
__global__ void __launch_bounds__(WARPS * 32, DEPTH_WHOLE == 4 ? 3 : 2)
gemm_small_whole_kernel(const void *__restrict__ Av, const bf16 *__restrict__ W,
                        void *__restrict__ Cv, int M, int N, int K, int lda, int ldw, int ldc, float eps) {
  static_assert(!NORMED || SPLIT == 1, "the normalised product is not split over a cluster");
  pdl_launch();
  const bf16 *A = reinterpret_cast<const bf16 *>(Av);
  constexpr int MROWS = MT * 8;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int nkb_all = (K + KB - 1) / KB;
  const int rank = SPLIT > 1 ? (int)(blockIdx.x % SPLIT) : 0;
  const int per = (nkb_all + SPLIT - 1) / SPLIT;
  const int kb_lo = rank * per, kb_hi = min(nkb_all, kb_lo + per);
  const int nkb = max(0, kb_hi - kb_lo);                  // K blocks of this CTA
  const int k_lo = kb_lo * KB;                            // first k of this CTA
  const int xrow = per * KB + XPAD;                       // staged row length (zero padded)
  bf16 *xs = reinterpret_cast<bf16 *>(smem_raw);          // [MROWS][xrow]
  float *red = reinterpret_cast<float *>(smem_raw + (((size_t)MROWS * xrow * sizeof(bf16)) + 127) / 128 * 128);
  float *part = red + WARPS * 16 * MROWS;                 // [16][MROWS]: this CTA's partial tile
  float *row_scale = part + 16 * MROWS;                   // [MROWS]: NORMED only

  const int n0 = (int)(blockIdx.x / SPLIT) * 16;
  const bf16 *w0 = W + (size_t)min(n0 + g, N - 1) * ldw;
  const bf16 *w1 = W + (size_t)min(n0 + g + 8, N - 1) * ldw;
  const int kw = 32 * warp + 8 * c;
  auto load_w = [&](uint4 (&dst)[2], int kb) {            // kb counts from this CTA's first block
    const int k = k_lo + kb * KB + kw;
    if (k < K) {
      dst[0] = ld_stream(w0 + k);
      dst[1] = ld_stream(w1 + k);
    } else {
      dst[0] = dst[1] = make_uint4(0, 0, 0, 0);
    }
  };
  // the weights do not depend on anything computed before: start their stream first
  uint4 wb[DEPTH_WHOLE][2];
#pragma unroll
  for (int d = 0; d < DEPTH_WHOLE; ++d)
    if (d < nkb) load_w(wb[d], d);
  pdl_wait();                            // the activations come from the kernel before

  // stage this CTA's columns of A: one warp per row, many copies in flight
  const int k_hi = min(K, k_lo + nkb * KB);               // one past this CTA's last k
  for (int r = warp; r < MROWS; r += WARPS) {
    bf16 *dst = xs + (size_t)r * xrow;
    if (r >= M) {
      for (int k = lane * 8; k < xrow; k += 256) *reinterpret_cast<uint4 *>(dst + k) = make_uint4(0, 0, 0, 0);
      if (NORMED && lane == 0) row_scale[r] = 0.f;
      continue;
    }
    if (NORMED) {
      // the row of the float stream: K a multiple of 8, so a lane takes 8 values at a time
      const float *x32 = reinterpret_cast<const float *>(Av) + (size_t)r * lda;
      float ss = 0.f;
      for (int k = lane * 8; k < K; k += 256) {
        const float4 a = *reinterpret_cast<const float4 *>(x32 + k);
        const float4 b = *reinterpret_cast<const float4 *>(x32 + k + 4);
        ss = fmaf(a.x, a.x, ss); ss = fmaf(a.y, a.y, ss); ss = fmaf(a.z, a.z, ss); ss = fmaf(a.w, a.w, ss);
        ss = fmaf(b.x, b.x, ss); ss = fmaf(b.y, b.y, ss); ss = fmaf(b.z, b.z, ss); ss = fmaf(b.w, b.w, ss);
        *reinterpret_cast<uint4 *>(dst + k) = make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w),
                                                         pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
      }
      for (int k = K + lane * 4; k < xrow; k += 128) *reinterpret_cast<uint2 *>(dst + k) = make_uint2(0, 0);
      ss = warp_sum(ss);
      if (lane == 0) row_scale[r] = 1.f / sqrtf(ss / (float)K + eps);
      continue;
    }
    const bf16 *x = A + (size_t)r * lda + k_lo;
    for (int k = lane * 8; k < k_hi - k_lo; k += 256) cp_async_16(smem_u32(dst + k), x + k);
    for (int k = max(0, k_hi - k_lo) + lane * 4; k < xrow; k += 128) *reinterpret_cast<uint2 *>(dst + k) = make_uint2(0, 0);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  float acc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
  for (int kb0 = 0; kb0 < nkb; kb0 += DEPTH_WHOLE) {
#pragma unroll
    for (int d = 0; d < DEPTH_WHOLE; ++d) {
      const int kb = kb0 + d;
      if (kb < nkb) {
        const bf16 *xb = xs + kb * KB + 32 * warp + 8 * c;
        const uint4 a_lo = wb[d][0], a_hi = wb[d][1];
        const uint32_t a1[4] = {a_lo.x, a_hi.x, a_lo.y, a_hi.y};
        const uint32_t a2[4] = {a_lo.z, a_hi.z, a_lo.w, a_hi.w};
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint4 xv = *reinterpret_cast<const uint4 *>(xb + (size_t)(8 * mt + g) * xrow);
          mma_bf16_16816(acc[mt], a1, xv.x, xv.y);
          mma_bf16_16816(acc[mt], a2, xv.z, xv.w);
        }
        if (kb + DEPTH_WHOLE < nkb) load_w(wb[d], kb + DEPTH_WHOLE);
      }
    }
  }
  // the 8 warps' partial sums -> shared memory, added in warp order
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    float *r0 = red + ((size_t)warp * 16 + g) * MROWS + 8 * mt + 2 * c;
    float *r1 = r0 + 8 * MROWS;
    r0[0] = acc[mt][0]; r0[1] = acc[mt][1];
    r1[0] = acc[mt][2]; r1[1] = acc[mt][3];
  }
  __syncthreads();
  if (SPLIT > 1) {
    // every CTA reduces its own warps; the first CTA of the cluster then adds the CTAs in order
    for (int i = threadIdx.x; i < 16 * MROWS; i += WARPS * 32) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) v += red[(size_t)w * 16 * MROWS + i];
      part[i] = v;
    }
    cooperative_groups::cluster_group cluster = cooperative_groups::this_cluster();
    cluster.sync();
    if (rank == 0) {
      for (int i = threadIdx.x; i < 16 * MROWS; i += WARPS * 32) {
        float v = part[i];
#pragma unroll
        for (int r = 1; r < SPLIT; ++r) v += cluster.map_shared_rank(part, r)[i];
        red[i] = v;                                   // the tile, as warp 0's partial; the others zero
#pragma unroll
        for (int w = 1; w < WARPS; ++w) red[(size_t)w * 16 * MROWS + i] = 0.f;
      }
    }
    cluster.sync();                                   // peers' memory stays alive until it was read
    if (rank != 0) return;
    __syncthreads();
  }
  if (EPI == EPI_SWIGLU_BF16) {
    for (int i = threadIdx.x; i < 8 * MROWS; i += WARPS * 32) {
      const int m = i / 8, r = i % 8;
      float gate = 0.f, up = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        gate += red[((size_t)w * 16 + r) * MROWS + m];
        up += red[((size_t)w * 16 + 8 + r) * MROWS + m];
      }
      if (NORMED) { gate *= row_scale[m]; up *= row_scale[m]; }
      const int col = (n0 >> 1) + r;
      if (m < M && n0 + 8 + r < N)
        ((bf16 *)Cv)[(size_t)m * ldc + col] = __float2bfloat16_rn((gate / (1.f + expf(-gate))) * up);
    }
  } else {
    for (int i = threadIdx.x; i < 16 * MROWS; i += WARPS * 32) {
      const int m = i / 16, r = i % 16;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) v += red[((size_t)w * 16 + r) * MROWS + m];
      if (NORMED) v *= row_scale[m];
      const int n = n0 + r;
      if (m < M && n < N) {
        const size_t o = (size_t)m * ldc + n;
        if (EPI == EPI_STORE_BF16) ((bf16 *)Cv)[o] = __float2bfloat16_rn(v);
        else if (EPI == EPI_STORE_F32) ((float *)Cv)[o] = v;
        else atomicAdd((float *)Cv + o, v);   // a reduction: one add per element and launch, no load on the path
      }
    }
  }
}

// ---- many tiles per CTA ----------------------------------------------------------------------
// For wide outputs with a long K (the layers of larger models) one 16-row tile per CTA is a
// poor unit: every CTA stages all of A first (half as many bytes as it then streams of W),
// the CTAs come in ragged rounds, and what a CTA keeps in flight is bounded by its registers.
// Here one CTA per SM takes a contiguous range of tiles, eight at a time, and walks over K in
// chunks of at most CB blocks: it stages a chunk of A once for the eight tiles (two buffers;
// the next chunk is fetched into registers while this one is in use) and streams that chunk's
// columns of W for each tile (16 rows x up to 4 KB contiguous per row), keeping the eight
// accumulators in registers.  The weights go through a ring of RING blocks in shared memory
// (16-byte cp.async; every thread reads back only what it copied itself, so the ring needs no
// barrier), which runs RING blocks = 128 KB ahead of the arithmetic across tiles, chunks and
// batches.  A thread sums its slice of K in the order of K and the 8 warps are added in
// order, exactly as in the kernels above: the result has the same bits.
template <int MT> struct StreamCfg {
  static constexpr int CB = 8 / MT;                 // K blocks per chunk: 8 rows x 2048 or 16 x 1024 columns
  static constexpr int MROWS = MT * 8;
  static constexpr int XROWS = CB * KB + XPAD;      // staged row length
  static constexpr int RING = 16;                   // blocks of W in flight: 16 rows x 512 bytes each
  static constexpr int BLOCK_BYTES = 16 * KB * 2;
  static constexpr size_t STAGE_BYTES = (size_t)2 * MROWS * XROWS * sizeof(bf16);
  static constexpr size_t RED_BYTES = (size_t)WARPS * 16 * MROWS * sizeof(float);
  static constexpr size_t TOTAL = STAGE_BYTES + RED_BYTES + (size_t)RING * BLOCK_BYTES;
};
constexpr int STREAM_BATCH = 8;                     // tiles whose accumulators a thread holds at once

template <int MT>
__global__ void __launch_bounds__(WARPS * 32, 1)
gemm_small_stream_kernel(const bf16 *__restrict__ A, const bf16 *__restrict__ W, void *__restrict__ Cv,
                         int M, int N, int K, int lda, int ldw, int ldc, int epi, int n_chunks, int kbc,
                         int tiles_per_cta) {
  pdl_launch();
  using C = StreamCfg<MT>;
  constexpr int MROWS = C::MROWS, XROWS = C::XROWS, RING = C::RING, G = STREAM_BATCH;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16 *xs = reinterpret_cast<bf16 *>(smem_raw);                        // [2][MROWS][XROWS]
  float *red = reinterpret_cast<float *>(smem_raw + C::STAGE_BYTES);    // [WARPS][16][MROWS]
  const uint32_t ring = smem_u32(smem_raw + C::STAGE_BYTES + C::RED_BYTES) + threadIdx.x * 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int kw = 32 * warp + 8 * c;
  const int n_tiles = (N + 15) / 16;
  const int t_begin = blockIdx.x * tiles_per_cta, t_end = min(n_tiles, t_begin + tiles_per_cta);

  // ---- the weight stream: blocks in the order (batch of 8 tiles, chunk, tile, block of the chunk)
  int p_tile0 = t_begin, p_chunk = 0, p_j = 0, p_d = 0;    // the block that is copied next
  uint32_t p_slot = 0;
  auto issue = [&]() {                                      // one block (or nothing), one group
    if (p_tile0 < t_end) {
      const int k = (p_chunk * kbc + p_d) * KB + kw;
      if (k < K) {
        const int n0 = (p_tile0 + p_j) * 16;
        cp_async_16(ring + p_slot * C::BLOCK_BYTES, W + (size_t)min(n0 + g, N - 1) * ldw + k);
        cp_async_16(ring + p_slot * C::BLOCK_BYTES + 4096, W + (size_t)min(n0 + g + 8, N - 1) * ldw + k);
      }
      if (++p_d == kbc) {
        p_d = 0;
        if (++p_j == min(G, t_end - p_tile0)) {          // the tiles of this batch that exist
          p_j = 0;
          if (++p_chunk == n_chunks) {
            p_chunk = 0;
            p_tile0 += G;
          }
        }
      }
    }
    cp_async_commit();
    p_slot = (p_slot + 1) % RING;
  };
  // the weights do not depend on anything computed before: start their stream first
#pragma unroll 1
  for (int i = 0; i < RING; ++i) issue();
  pdl_wait();                            // the activations come from the kernel before

  // rows past M of both buffers stay zero
  for (int i = threadIdx.x; i < 2 * MROWS * (XROWS / 8); i += WARPS * 32) {
    const int r = (i / (XROWS / 8)) % MROWS;
    if (r >= M) *reinterpret_cast<uint4 *>(xs + (size_t)i * 8) = make_uint4(0, 0, 0, 0);
  }
  // a chunk of A: one 16-byte piece per thread and row, through registers
  const bool stager = (int)threadIdx.x < kbc * (KB / 8);
  uint4 areg[MROWS];
  auto fetch_a = [&](int chunk) {
    const int k = chunk * kbc * KB + threadIdx.x * 8;
#pragma unroll
    for (int r = 0; r < MROWS; ++r)
      areg[r] = (stager && r < M && k < K) ? *reinterpret_cast<const uint4 *>(A + (size_t)r * lda + k)
                                           : make_uint4(0, 0, 0, 0);
  };
  auto store_a = [&](int buf) {
    if (stager) {
      bf16 *dst = xs + (size_t)buf * MROWS * XROWS + threadIdx.x * 8;
#pragma unroll
      for (int r = 0; r < MROWS; ++r)
        if (r < M) *reinterpret_cast<uint4 *>(dst + (size_t)r * XROWS) = areg[r];
    }
  };

  uint32_t c_slot = 0;                                  // the ring slot that is consumed next
  for (int tile0 = t_begin; tile0 < t_end; tile0 += G) {
    float acc[G][MT][4];
#pragma unroll
    for (int j = 0; j < G; ++j)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) acc[j][mt][0] = acc[j][mt][1] = acc[j][mt][2] = acc[j][mt][3] = 0.f;
    fetch_a(0);
    store_a(0);
    for (int chunk = 0; chunk < n_chunks; ++chunk) {
      __syncthreads();                               // this chunk of A is in place; the other buffer is free
      if (chunk + 1 < n_chunks) fetch_a(chunk + 1);
      const bf16 *xc = xs + (size_t)(chunk & 1) * MROWS * XROWS + kw;
#pragma unroll
      for (int j = 0; j < G; ++j) {
        if (tile0 + j < t_end) {
          for (int d = 0; d < kbc; ++d) {
            cp_async_wait<RING - 1>();               // this thread's copies of the block have landed
            uint4 a_lo = make_uint4(0, 0, 0, 0), a_hi = a_lo;
            if ((chunk * kbc + d) * KB + kw < K) {
              asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n"
                           : "=r"(a_lo.x), "=r"(a_lo.y), "=r"(a_lo.z), "=r"(a_lo.w)
                           : "r"(ring + c_slot * C::BLOCK_BYTES));
              asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n"
                           : "=r"(a_hi.x), "=r"(a_hi.y), "=r"(a_hi.z), "=r"(a_hi.w)
                           : "r"(ring + c_slot * C::BLOCK_BYTES + 4096));
            }
            c_slot = (c_slot + 1) % RING;
            const uint32_t a1[4] = {a_lo.x, a_hi.x, a_lo.y, a_hi.y};
            const uint32_t a2[4] = {a_lo.z, a_hi.z, a_lo.w, a_hi.w};
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const uint4 xv = *reinterpret_cast<const uint4 *>(xc + d * KB + (size_t)(8 * mt + g) * XROWS);
              mma_bf16_16816(acc[j][mt], a1, xv.x, xv.y);
              mma_bf16_16816(acc[j][mt], a2, xv.z, xv.w);
            }
            issue();                                 // the slot just read is filled again
          }
        }
      }
      if (chunk + 1 < n_chunks) store_a((chunk + 1) & 1);
    }

    // per tile: the 8 warps' partial sums -> shared memory, added in warp order
#pragma unroll
    for (int j = 0; j < G; ++j) {
      if (tile0 + j >= t_end) break;
      __syncthreads();                               // `red` is free (and, for j = 0, A's buffers are)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        float *r0 = red + ((size_t)warp * 16 + g) * MROWS + 8 * mt + 2 * c;
        float *r1 = r0 + 8 * MROWS;
        r0[0] = acc[j][mt][0]; r0[1] = acc[j][mt][1];
        r1[0] = acc[j][mt][2]; r1[1] = acc[j][mt][3];
      }
      __syncthreads();
      const int n0 = (tile0 + j) * 16;
      if (epi == EPI_SWIGLU_BF16) {
        for (int i = threadIdx.x; i < 8 * MROWS; i += WARPS * 32) {
          const int m = i / 8, r = i % 8;
          float gate = 0.f, up = 0.f;
#pragma unroll
          for (int w = 0; w < WARPS; ++w) {
            gate += red[((size_t)w * 16 + r) * MROWS + m];
            up += red[((size_t)w * 16 + 8 + r) * MROWS + m];
          }
          if (m < M && n0 + 8 + r < N)
            ((bf16 *)Cv)[(size_t)m * ldc + (n0 >> 1) + r] = __float2bfloat16_rn((gate / (1.f + expf(-gate))) * up);
        }
      } else {
        for (int i = threadIdx.x; i < 16 * MROWS; i += WARPS * 32) {
          const int m = i / 16, r = i % 16;
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < WARPS; ++w) v += red[((size_t)w * 16 + r) * MROWS + m];
          const int n = n0 + r;
          if (m < M && n < N) {
            const size_t o = (size_t)m * ldc + n;
            if (epi == EPI_STORE_BF16) ((bf16 *)Cv)[o] = __float2bfloat16_rn(v);
            else if (epi == EPI_STORE_F32) ((float *)Cv)[o] = v;
            else atomicAdd((float *)Cv + o, v);   // a reduction: one add per element and launch
          }
        }
      }
    }
    __syncthreads();                                 // before the next batch stages A
  }
  cp_async_wait<0>();
}

// shared memory the whole-A kernel needs, or 0 if the case does not fit
static size_t whole_smem(int mrows, int K, int split = 1) {
  const int nkb = (K + KB - 1) / KB, per = (nkb + split - 1) / split;
  const size_t stage = ((size_t)mrows * (per * KB + XPAD) * sizeof(bf16) + 127) / 128 * 128;
  const size_t red = ((size_t)(WARPS + 1) * 16 * mrows + mrows) * sizeof(float);    // + a factor per row
  const size_t need = stage + red;
  return need <= 200 * 1024 ? need : 0;
}

// CTAs per 16-row tile: narrow outputs with a long K are split over a cluster
static int pick_split(int N, int K) {
  const int n_tiles = (N + 15) / 16, nkb = (K + KB - 1) / KB;
  if (n_tiles <= 96 && nkb >= 12) return 4;      // measured: K = 2048 is faster unsplit, K = 3072 split
  if (n_tiles <= 160 && nkb >= 10) return 2;
  return 1;
}

// the split that is built for the case: a CTA of a split product keeps at most 4 blocks of K
static int final_split(int N, int K) {
  const int nkb = (K + KB - 1) / KB, s = pick_split(N, K);
  if (s == 4 && (nkb + 3) / 4 <= 4) return 4;
  if (s >= 2 && (nkb + 1) / 2 <= 4) return 2;
  return 1;
}

template <int MT, int DEPTH_WHOLE, int SPLIT>
static int launch_whole_depth(const void *A, const void *W, void *C, int M, int N, int K, int lda, int ldw,
                              int ldc, int epi, cudaStream_t stream) {
  const int smem = (int)whole_smem(MT * 8, K, SPLIT);
  const int n_tiles = (N + 15) / 16;
  const unsigned grid = (unsigned)(n_tiles * SPLIT);
#define G2B_LAUNCH(E)                                                                            \
  do {                                                                                           \
    static G2bPerDevice configured;                                                              \
    const int cfg_dev = g2b_current_device();                                                    \
    if (cfg_dev < 0 || configured.value[cfg_dev] < smem) {                                       \
      cudaError_t e = cudaFuncSetAttribute(gemm_small_whole_kernel<MT, E, DEPTH_WHOLE, SPLIT>,       \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, smem);   \
      if (e != cudaSuccess) G2B_REFUSE("gemm_small: shared memory: %s", cudaGetErrorString(e));  \
      if (cfg_dev >= 0) configured.value[cfg_dev] = smem;                                        \
    }                                                                                            \
    g2b_launch_cluster(gemm_small_whole_kernel<MT, E, DEPTH_WHOLE, SPLIT>, dim3(grid),           \
                       dim3(WARPS * 32), smem, stream, (unsigned)SPLIT, (const void *)A,         \
                       (const bf16 *)W, C, M, N, K, lda, ldw, ldc, 0.f);                         \
  } while (0)
  switch (epi) {
    case EPI_STORE_BF16: G2B_LAUNCH(EPI_STORE_BF16); break;
    case EPI_STORE_F32: G2B_LAUNCH(EPI_STORE_F32); break;
    case EPI_ACCUM_F32: G2B_LAUNCH(EPI_ACCUM_F32); break;
    case EPI_SWIGLU_BF16: G2B_LAUNCH(EPI_SWIGLU_BF16); break;
    default: G2B_REFUSE("gemm_small: unknown epilogue %d", epi);
  }
#undef G2B_LAUNCH
  return g2b_check_launch("gemm_small_whole");
}

template <int MT>
static int launch_whole(const void *A, const void *W, void *C, int M, int N, int K, int lda, int ldw, int ldc,
                        int epi, cudaStream_t stream) {
  const int nkb = (K + KB - 1) / KB;
  const int split = final_split(N, K);
  if (split == 4) return launch_whole_depth<MT, 4, 4>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
  if (split == 2) return launch_whole_depth<MT, 4, 2>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
  if (nkb <= 4) return launch_whole_depth<MT, 4, 1>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
  return launch_whole_depth<MT, 8, 1>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
}

template <int MT>
static int launch_mt(const void *A, const void *W, void *C, int M, int N, int K, int lda, int ldw,
                     int ldc, int epi, cudaStream_t stream) {
  constexpr int MROWS = MT * 8;
  const size_t stage = (size_t)2 * MROWS * XROW * sizeof(bf16);
  const size_t red = (size_t)WARPS * 16 * MROWS * sizeof(float);
  const int smem = (int)(stage > red ? stage : red);
  const unsigned grid = (unsigned)((N + 15) / 16);
#define G2B_LAUNCH(E)                                                                            \
  do {                                                                                           \
    static G2bPerDevice configured;                                                              \
    const int cfg_dev = g2b_current_device();                                                    \
    if (cfg_dev < 0 || !configured.value[cfg_dev]) {                                             \
      cudaError_t e = cudaFuncSetAttribute(gemm_small_kernel<MT, E>,                             \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, smem);   \
      if (e != cudaSuccess) G2B_REFUSE("gemm_small: shared memory: %s", cudaGetErrorString(e));  \
      if (cfg_dev >= 0) configured.value[cfg_dev] = 1;                                           \
    }                                                                                            \
    g2b_launch(gemm_small_kernel<MT, E>, dim3(grid), dim3(WARPS * 32), smem, stream,                                 \
        (const bf16 *)A, (const bf16 *)W, C, M, N, K, lda, ldw, ldc);                            \
  } while (0)
  switch (epi) {
    case EPI_STORE_BF16: G2B_LAUNCH(EPI_STORE_BF16); break;
    case EPI_STORE_F32: G2B_LAUNCH(EPI_STORE_F32); break;
    case EPI_ACCUM_F32: G2B_LAUNCH(EPI_ACCUM_F32); break;
    case EPI_SWIGLU_BF16: G2B_LAUNCH(EPI_SWIGLU_BF16); break;
    default: G2B_REFUSE("gemm_small: unknown epilogue %d", epi);
  }
#undef G2B_LAUNCH
  return g2b_check_launch("gemm_small");
}

// The product of RMS-normalised rows of the float stream (see NORMED above): whole-A kernel,
// one CTA per tile.
template <int MT, int DEPTH_WHOLE>
static int launch_normed(const float *X, const void *W, void *C, int M, int N, int K, int ldx, int ldw,
                         int ldc, int epi, float eps, cudaStream_t stream) {
  const int smem = (int)whole_smem(MT * 8, K, 1);
  const unsigned grid = (unsigned)((N + 15) / 16);
#define G2B_LAUNCH(E)                                                                            \
  do {                                                                                           \
    static G2bPerDevice configured;                                                              \
    const int cfg_dev = g2b_current_device();                                                    \
    if (cfg_dev < 0 || configured.value[cfg_dev] < smem) {                                       \
      cudaError_t e = cudaFuncSetAttribute(gemm_small_whole_kernel<MT, E, DEPTH_WHOLE, 1, true>, \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, smem);   \
      if (e != cudaSuccess) G2B_REFUSE("gemm_small: shared memory: %s", cudaGetErrorString(e));  \
      if (cfg_dev >= 0) configured.value[cfg_dev] = smem;                                        \
    }                                                                                            \
    g2b_launch(gemm_small_whole_kernel<MT, E, DEPTH_WHOLE, 1, true>, dim3(grid), dim3(WARPS * 32), smem, \
               stream, (const void *)X, (const bf16 *)W, C, M, N, K, ldx, ldw, ldc, eps);        \
  } while (0)
  switch (epi) {
    case EPI_STORE_BF16: G2B_LAUNCH(EPI_STORE_BF16); break;
    case EPI_STORE_F32: G2B_LAUNCH(EPI_STORE_F32); break;
    case EPI_SWIGLU_BF16: G2B_LAUNCH(EPI_SWIGLU_BF16); break;
    default: G2B_REFUSE("gemm_small_normed: epilogue %d (store or SiLU gate only)", epi);
  }
#undef G2B_LAUNCH
  return g2b_check_launch("gemm_small_normed");
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

// Whether the many-tiles kernel takes the case: up to 8 rows (with more, the tcgen05 kernel that
// splits K over a cluster is faster against weights of this size), enough tiles to fill the GPU
// by themselves, and a K of 2,048 or more (at K = 1,024 a tile is four blocks, and the per-tile
// sum over the warps weighs more than what the shared staging saves: 70 against 59 us for a
// vocabulary of 151,936).
static bool stream_case(int M, int N, int K) {
  const int n_tiles = (N + 15) / 16, nkb = (K + KB - 1) / KB;
  return M <= 8 && n_tiles >= sm_count() && nkb >= 8;
}

template <int MT>
static int launch_stream(const void *A, const void *W, void *C, int M, int N, int K, int lda, int ldw, int ldc,
                         int epi, cudaStream_t stream) {
  if (epi < EPI_STORE_BF16 || epi > EPI_SWIGLU_BF16) G2B_REFUSE("gemm_small: unknown epilogue %d", epi);
  constexpr int CB = StreamCfg<MT>::CB;
  const int smem = (int)StreamCfg<MT>::TOTAL;
  static G2bPerDevice configured;
  const int cfg_dev = g2b_current_device();
  if (cfg_dev < 0 || !configured.value[cfg_dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_small_stream_kernel<MT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) G2B_REFUSE("gemm_small: shared memory: %s", cudaGetErrorString(e));
    if (cfg_dev >= 0) configured.value[cfg_dev] = 1;
  }
  const int n_tiles = (N + 15) / 16, nkb = (K + KB - 1) / KB;
  const int n_chunks = (nkb + CB - 1) / CB, kbc = (nkb + n_chunks - 1) / n_chunks;
  const int per = (n_tiles + sm_count() - 1) / sm_count();          // tiles per CTA: the same for (almost) all
  const unsigned grid = (unsigned)((n_tiles + per - 1) / per);
  g2b_launch(gemm_small_stream_kernel<MT>, dim3(grid), dim3(WARPS * 32), smem, stream, (const bf16 *)A,
             (const bf16 *)W, C, M, N, K, lda, ldw, ldc, epi, n_chunks, kbc, per);
  return g2b_check_launch("gemm_small_stream");
}

// A [M,K] and W [N,K] bfloat16 with unit inner stride; rows 16-byte aligned.
// epi: 0 store bfloat16, 1 store float, 2 add into float, 3 SiLU gate (C is [M, N/2] bfloat16;
// N must be a multiple of 16).
extern "C" int g2b_gemm_small(const void *A, const void *W, void *C, int M, int N, int K, int lda,
                              int ldw, int ldc, int epi, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64) G2B_REFUSE("gemm_small: M=%d (at most 64 rows)", M);
  if (K <= 0 || K % 8 || lda % 8 || ldw % 8)
    G2B_REFUSE("gemm_small: K=%d and the row strides (%d, %d) must be multiples of 8", K, lda, ldw);
  if (((uintptr_t)A | (uintptr_t)W) & 15) G2B_REFUSE("gemm_small: operands must be 16-byte aligned");
  if (epi == EPI_SWIGLU_BF16 && N % 16) G2B_REFUSE("gemm_small: gated output needs N %% 16 == 0, N=%d", N);
  if (stream_case(M, N, K)) return launch_stream<1>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
  const int mrows = M <= 8 ? 8 : (M <= 16 ? 16 : (M <= 32 ? 32 : 64));
  if (whole_smem(mrows, K, final_split(N, K))) {
    if (M <= 8) return launch_whole<1>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
    if (M <= 16) return launch_whole<2>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
    if (M <= 32) return launch_whole<4>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
    return launch_whole<8>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
  }
  if (M <= 8) return launch_mt<1>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
  if (M <= 16) return launch_mt<2>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
  if (M <= 32) return launch_mt<4>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
  return launch_mt<8>(A, W, C, M, N, K, lda, ldw, ldc, epi, stream);
}

// Whether g2b_gemm_small_normed takes the case: up to 16 rows, the whole of A in shared memory,
// an output wide enough that K is not split over a cluster, and not the shapes that the
// many-tiles kernel is faster for.
extern "C" int g2b_gemm_small_normed_takes(int M, int N, int K) {
  if (M <= 0 || M > 16 || N <= 0 || K <= 0 || K % 8) return 0;
  if (stream_case(M, N, K)) return 0;
  return whole_smem(M <= 8 ? 8 : 16, K, 1) != 0 && final_split(N, K) == 1;
}

// C = norm(X) . W^T for X [M, K] float (the residual stream), norm(x) = x / sqrt(mean(x^2) + eps)
// without a per-channel weight; W [N, K] bfloat16.  epi as g2b_gemm_small's, without 2.
extern "C" int g2b_gemm_small_normed(const float *X, const void *W, void *C, int M, int N, int K, int ldx,
                                     int ldw, int ldc, int epi, float eps, cudaStream_t stream) {
  if (!g2b_gemm_small_normed_takes(M, N, K)) G2B_REFUSE("gemm_small_normed: M=%d N=%d K=%d is not taken", M, N, K);
  if (ldx % 4 || ldw % 8) G2B_REFUSE("gemm_small_normed: row strides (%d, %d)", ldx, ldw);
  if (((uintptr_t)X | (uintptr_t)W) & 15) G2B_REFUSE("gemm_small_normed: operands must be 16-byte aligned");
  if (epi == EPI_SWIGLU_BF16 && N % 16) G2B_REFUSE("gemm_small_normed: gated output needs N %% 16 == 0, N=%d", N);
  const int nkb = (K + KB - 1) / KB;
  if (M <= 8) {
    if (nkb <= 4) return launch_normed<1, 4>(X, W, C, M, N, K, ldx, ldw, ldc, epi, eps, stream);
    return launch_normed<1, 8>(X, W, C, M, N, K, ldx, ldw, ldc, epi, eps, stream);
  }
  if (nkb <= 4) return launch_normed<2, 4>(X, W, C, M, N, K, ldx, ldw, ldc, epi, eps, stream);
  return launch_normed<2, 8>(X, W, C, M, N, K, ldx, ldw, ldc, epi, eps, stream);
}
