// Memory-bound kernels of the step: embedding rows, RMSNorm (optionally on gathered
// rows), fused per-head RMSNorm + half-split rotation + cache write, the cache write
// alone, and the SiLU gate.  All statistics, angles and products are 32-bit.
//
// Formulas (paths relative to AnonymoDGH/gguf2bin):
//   embedding      src/l5_model.c:488-491
//   rmsnorm        src/l3_math.c:34-36,49      o_j = (w_j * x_j) * 1/sqrt(sum x^2 / n + eps)
//   per-head norm  src/l3_math.c:107-114
//   rotation       src/l3_math.c:84-102        pairs (j, j+half), ang = pos * freq_j
//   cache write    src/l5_model.c:232-247      K after norm and rotation, V raw
//   SiLU gate      src/l3_math.c:57-62, src/l5_model.c:594-595
#include "common.cuh"

G2B_DEFINE_LAST_ERROR

// ---------------------------------------------------------------------------
// embedding: out[t, :] = table[ids[t], :]   (out is the 32-bit residual stream)
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void embed_rows_kernel(const TW *__restrict__ table, const int *__restrict__ ids,
                                  float *__restrict__ out, int H, int V) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  const bool ok = (id >= 0 && id < V);
  if (!ok) id = 0;                                   // host validates ids; never read outside
  const TW *row = table + (size_t)id * H;
  float *o = out + (size_t)t * H;
  for (int j = threadIdx.x; j < H; j += blockDim.x) o[j] = ok ? to_f32(row[j]) : 0.f;
}

extern "C" int g2b_embed_rows(const void *table, int table_dtype, const int *ids, float *out,
                              int T, int H, int V, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || V <= 0) G2B_REFUSE("embed_rows: bad sizes H=%d V=%d", H, V);
  const int threads = H >= 256 ? 256 : 64;
  if (table_dtype == G2B_F32)
    g2b_launch(embed_rows_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float *)table, ids, out, H, V);
  else if (table_dtype == G2B_BF16)
    g2b_launch(embed_rows_kernel<bf16>, dim3(T), dim3(threads), 0, stream, (const bf16 *)table, ids, out, H, V);
  else
    G2B_REFUSE("embed_rows: unknown table dtype %d", table_dtype);
  return g2b_check_launch("embed_rows");
}

// ---------------------------------------------------------------------------
// rmsnorm over rows of the 32-bit stream; rows == nullptr means rows 0..n_rows-1;
// w == nullptr means no per-channel weight (it was multiplied into the next matrix)
// ---------------------------------------------------------------------------
template <typename TO>
__global__ void rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ w,
                               const int *__restrict__ rows, TO *__restrict__ out, int H,
                               float eps) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const float *xr = x + (size_t)(rows ? rows[r] : r) * H;
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float v = xr[j];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)H + eps);
  TO *o = out + (size_t)r * H;
  for (int j = threadIdx.x; j < H; j += blockDim.x) o[j] = from_f32<TO>(((w ? w[j] : 1.f) * xr[j]) * inv);
}

__device__ __forceinline__ void store4(float *p, float a, float b, float c, float d) {
  *reinterpret_cast<float4 *>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(bf16 *p, float a, float b, float c, float d) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162 *>(&raw.x) = __floats2bfloat162_rn(a, b);
  *reinterpret_cast<__nv_bfloat162 *>(&raw.y) = __floats2bfloat162_rn(c, d);
  *reinterpret_cast<uint2 *>(p) = raw;
}

// one warp per row, 16-byte loads, eight of them in flight per lane, four outputs per store; rows
// of up to 1,024 elements stay in registers between the two passes; H a multiple of 4
template <typename TO>
__global__ void __launch_bounds__(128)
rmsnorm_rows_kernel(const float *__restrict__ x, const float *__restrict__ w,
                    const int *__restrict__ rows, TO *__restrict__ out, int n_rows, int H,
                    float eps) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const float *xr = x + (size_t)(rows ? rows[r] : r) * H;
  float ss = 0.f;
  if (H <= 1024) {
    float4 v[8], g[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int k = lane * 4 + 128 * i;
      v[i] = k < H ? *reinterpret_cast<const float4 *>(xr + k) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int k = lane * 4 + 128 * i;
      g[i] = !w ? make_float4(1.f, 1.f, 1.f, 1.f)
                : (k < H ? *reinterpret_cast<const float4 *>(w + k) : make_float4(0.f, 0.f, 0.f, 0.f));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
      ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)H + eps);
    TO *o = out + (size_t)r * H;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int k = lane * 4 + 128 * i;
      if (k < H)
        store4(o + k, (g[i].x * v[i].x) * inv, (g[i].y * v[i].y) * inv, (g[i].z * v[i].z) * inv,
               (g[i].w * v[i].w) * inv);
    }
    return;
  }
  for (int k0 = lane * 4; k0 < H; k0 += 128 * 8) {
    float4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int k = k0 + 128 * i;
      v[i] = k < H ? *reinterpret_cast<const float4 *>(xr + k) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
      ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
    }
  }
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)H + eps);
  TO *o = out + (size_t)r * H;
  for (int k0 = lane * 4; k0 < H; k0 += 128 * 4) {
    float4 v[4], g[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + 128 * i;
      if (k < H) {
        v[i] = *reinterpret_cast<const float4 *>(xr + k);
        g[i] = w ? *reinterpret_cast<const float4 *>(w + k) : make_float4(1.f, 1.f, 1.f, 1.f);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + 128 * i;
      if (k < H)
        store4(o + k, (g[i].x * v[i].x) * inv, (g[i].y * v[i].y) * inv, (g[i].z * v[i].z) * inv,
               (g[i].w * v[i].w) * inv);
    }
  }
}

// one block of 256 threads per row for rows of 1,025 to 8,192 elements: the whole row and its
// weights are fetched at once (up to eight 16-byte loads each per thread) and stay in registers
// between the sum and the output; H a multiple of 4
template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_block_kernel(const float *__restrict__ x, const float *__restrict__ w,
                     const int *__restrict__ rows, TO *__restrict__ out, int H, float eps) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const float *xr = x + (size_t)(rows ? rows[r] : r) * H;
  float4 v[8], g[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int k = threadIdx.x * 4 + 1024 * i;
    v[i] = k < H ? *reinterpret_cast<const float4 *>(xr + k) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int k = threadIdx.x * 4 + 1024 * i;
    g[i] = !w ? make_float4(1.f, 1.f, 1.f, 1.f)
              : (k < H ? *reinterpret_cast<const float4 *>(w + k) : make_float4(0.f, 0.f, 0.f, 0.f));
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
    ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)H + eps);
  TO *o = out + (size_t)r * H;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int k = threadIdx.x * 4 + 1024 * i;
    if (k < H)
      store4(o + k, (g[i].x * v[i].x) * inv, (g[i].y * v[i].y) * inv, (g[i].z * v[i].z) * inv,
             (g[i].w * v[i].w) * inv);
  }
}

extern "C" int g2b_rmsnorm(const float *x, const float *w, const int *rows, int n_rows, int H,
                           float eps, void *out, int out_dtype, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (H <= 0) G2B_REFUSE("rmsnorm: bad width %d", H);
  if (H % 4 == 0 && H >= 128 && ((((uintptr_t)x) | ((uintptr_t)w) | ((uintptr_t)out)) & 15) == 0 &&
      (out_dtype == G2B_F32 || out_dtype == G2B_BF16)) {
    if (H > 1024 && H <= 8192) {
      if (out_dtype == G2B_F32)
        g2b_launch(rmsnorm_block_kernel<float>, dim3((unsigned)n_rows), dim3(256), 0, stream, x, w, rows, (float *)out, H, eps);
      else
        g2b_launch(rmsnorm_block_kernel<bf16>, dim3((unsigned)n_rows), dim3(256), 0, stream, x, w, rows, (bf16 *)out, H, eps);
      return g2b_check_launch("rmsnorm");
    }
    const unsigned blocks = (unsigned)((n_rows + 3) / 4);
    if (out_dtype == G2B_F32)
      g2b_launch(rmsnorm_rows_kernel<float>, dim3(blocks), dim3(128), 0, stream, x, w, rows, (float *)out, n_rows, H, eps);
    else
      g2b_launch(rmsnorm_rows_kernel<bf16>, dim3(blocks), dim3(128), 0, stream, x, w, rows, (bf16 *)out, n_rows, H, eps);
    return g2b_check_launch("rmsnorm");
  }
  const int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 32);
  if (out_dtype == G2B_F32)
    g2b_launch(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, w, rows, (float *)out, H, eps);
  else if (out_dtype == G2B_BF16)
    g2b_launch(rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, x, w, rows, (bf16 *)out, H, eps);
  else
    G2B_REFUSE("rmsnorm: unknown output dtype %d", out_dtype);
  return g2b_check_launch("rmsnorm");
}

// ---------------------------------------------------------------------------
// per-head norm + rotation + cache write.  One warp per (token, head) of the fused
// projection output qkv[t] = [q heads | k heads | v heads].
//   q heads: norm (if q_w), rotate (if a table is given)  -> q_out[t, h*hd + j]
//   k heads: norm (if k_w), rotate (if a table is given)  -> cache K, or k_out when given
//   v heads: copied                                -> cache V, or v_out when given
// Cache of one layer: [n_pages][2][nkv][page_size][hd]; the page of position p of
// sequence b is page_table[b*P + p/page_size].
// ---------------------------------------------------------------------------
#define QKN_MAX_HD 512
#define QKN_WARPS 4

// cos and sin of pos * inv_freq[j] for every token of the step, once per step: all layers
// with the same frequencies read the same table.  table[t * half + j] = (cos, sin).
__global__ void rope_table_kernel(const int *__restrict__ tok_pos, const float *__restrict__ inv_freq,
                                  float2 *__restrict__ table, int T_tokens, int half) {
  pdl_launch();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)T_tokens * half) return;
  const int t = (int)(i / half), j = (int)(i % half);
  float sn, c;
  sincosf((float)tok_pos[t] * inv_freq[j], &sn, &c);
  table[i] = make_float2(c, sn);
}

extern "C" int g2b_rope_table(const int *tok_pos, const float *inv_freq, float *table, int T_tokens,
                              int half, cudaStream_t stream) {
  if (T_tokens <= 0 || half <= 0) return 0;
  const long long n = (long long)T_tokens * half;
  g2b_launch(rope_table_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, tok_pos, inv_freq,
             (float2 *)table, T_tokens, half);
  return g2b_check_launch("rope_table");
}

// Head sizes 2 * E * LPH (LPH a power of two up to 32, E = 4 or 8) with the rotation over the
// whole head: LPH lanes share a head, so a warp works on 32 / LPH heads of one token at once.
// A lane holds E consecutive elements of the first half and their rotation partners in the
// second half, loaded and stored as vectors; everything stays in registers.  E = 4 gives a
// decode step more lanes per head (shorter chains); E = 8 moves 16 bytes per load for prompts.
#define QKN_FAST_WARPS 8

template <int E> __device__ __forceinline__ void ldE(const bf16 *p, float (&v)[E]) {
  if constexpr (E == 8) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[i]));
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  } else {
    const uint2 raw = *reinterpret_cast<const uint2 *>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.y));
    v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
  }
}
template <int E> __device__ __forceinline__ void ldE(const float *p, float (&v)[E]) {
#pragma unroll
  for (int i = 0; i < E; i += 4) {
    const float4 raw = *reinterpret_cast<const float4 *>(p + i);
    v[i] = raw.x; v[i + 1] = raw.y; v[i + 2] = raw.z; v[i + 3] = raw.w;
  }
}
template <int E> __device__ __forceinline__ void stE(bf16 *p, const float (&v)[E]) {
  uint32_t w[E / 2];
#pragma unroll
  for (int i = 0; i < E / 2; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t *>(&h);
  }
  if constexpr (E == 8) *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  else *reinterpret_cast<uint2 *>(p) = make_uint2(w[0], w[1]);
}
template <int E> __device__ __forceinline__ void stE(float *p, const float (&v)[E]) {
#pragma unroll
  for (int i = 0; i < E; i += 4) *reinterpret_cast<float4 *>(p + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
}

template <typename T, int LPH, int E>
__global__ void __launch_bounds__(QKN_FAST_WARPS * 32)
qknorm_rope_fast_kernel(
    const T *__restrict__ qkv, int T_tokens, int nh, int nkv,
    const float *__restrict__ q_w, const float *__restrict__ k_w, float eps,
    const float2 *__restrict__ rope,
    const int *__restrict__ tok_pos, const int *__restrict__ tok_seq,
    const int *__restrict__ page_table, int P, T *__restrict__ cache, int page_size,
    T *__restrict__ q_out, T *__restrict__ k_out, T *__restrict__ v_out) {
  pdl_launch();
  pdl_wait();
  constexpr int HPW = 32 / LPH, HD = 2 * E * LPH, HH = E * LPH;
  const unsigned warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned heads = nh + 2 * nkv;
  const unsigned groups = (heads + HPW - 1) / HPW;
  const unsigned item = blockIdx.x * QKN_FAST_WARPS + warp;
  if (item >= (unsigned)T_tokens * groups) return;
  const unsigned t = item / groups;
  const unsigned h = (item - t * groups) * HPW + lane / LPH;
  const bool valid = h < heads;
  const unsigned hc = valid ? h : heads - 1;
  const int j = E * (lane % LPH);
  const T *src = qkv + ((size_t)t * heads + hc) * HD;
  float a[E], b[E];
  ldE<E>(src + j, a);
  ldE<E>(src + HH + j, b);
  const int kind = hc < (unsigned)nh ? 0 : (hc < (unsigned)(nh + nkv) ? 1 : 2);     // q, k, v
  const float *w = kind == 0 ? q_w : (kind == 1 ? k_w : nullptr);
  T *dst;
  if (kind == 0) {
    dst = q_out + ((size_t)t * nh + hc) * HD;
  } else {
    const unsigned kvh = kind == 1 ? hc - nh : hc - nh - nkv;
    T *flat = kind == 1 ? k_out : v_out;
    if (flat) {
      dst = flat + ((size_t)t * nkv + kvh) * HD;
    } else {
      const int pos = tok_pos[t];
      const int page = page_table[(size_t)tok_seq[t] * P + pos / page_size];
      dst = cache + ((((size_t)page * 2 + (kind - 1)) * nkv + kvh) * page_size + pos % page_size) * HD;
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < E; ++i) {
    ss = fmaf(a[i], a[i], ss);
    ss = fmaf(b[i], b[i], ss);
  }
#pragma unroll
  for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (w) {
    const float inv = 1.f / sqrtf(ss / (float)HD + eps);
    float wa[E], wb[E];
    ldE<E>(w + j, wa);
    ldE<E>(w + HH + j, wb);
#pragma unroll
    for (int i = 0; i < E; ++i) {
      a[i] = (wa[i] * a[i]) * inv;
      b[i] = (wb[i] * b[i]) * inv;
    }
  }
  if (rope && kind != 2) {
    const float2 *cs = rope + (size_t)t * HH + j;
#pragma unroll
    for (int i = 0; i < E; i += 2) {
      const float4 r = *reinterpret_cast<const float4 *>(cs + i);      // (cos, sin) of j+i, j+i+1
      const float a0 = a[i], b0 = b[i], a1 = a[i + 1], b1 = b[i + 1];
      a[i] = a0 * r.x - b0 * r.y;
      b[i] = a0 * r.y + b0 * r.x;
      a[i + 1] = a1 * r.z - b1 * r.w;
      b[i + 1] = a1 * r.w + b1 * r.z;
    }
  }
  if (valid) {
    stE<E>(dst + j, a);
    stE<E>(dst + HH + j, b);
  }
}

// Every other head size and a rotation over part of the head: one warp per (token, head),
// the head staged in shared memory.
template <typename T>
__global__ void __launch_bounds__(QKN_WARPS * 32)
qknorm_rope_cache_kernel(
    const T *__restrict__ qkv, int T_tokens, int nh, int nkv, int hd,
    const float *__restrict__ q_w, const float *__restrict__ k_w, float eps,
    const float2 *__restrict__ rope, int rot_dim,
    const int *__restrict__ tok_pos, const int *__restrict__ tok_seq,
    const int *__restrict__ page_table, int P, T *__restrict__ cache, int page_size,
    T *__restrict__ q_out, T *__restrict__ k_out, T *__restrict__ v_out) {
  pdl_launch();
  pdl_wait();
  __shared__ float buf[QKN_WARPS][QKN_MAX_HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = nh + 2 * nkv;
  const long long item = (long long)blockIdx.x * QKN_WARPS + warp;
  if (item >= (long long)T_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads);
  const int half = rot_dim >> 1;
  const T *src = qkv + (size_t)t * heads * hd + (size_t)h * hd;
  const int kind = h < nh ? 0 : (h < nh + nkv ? 1 : 2);
  const float *w = kind == 0 ? q_w : (kind == 1 ? k_w : nullptr);
  const float2 *cs = (rope && kind != 2) ? rope + (size_t)t * half : nullptr;
  T *dst;
  if (kind == 0) {
    dst = q_out + (size_t)t * nh * hd + (size_t)h * hd;
  } else {
    const int kvh = kind == 1 ? h - nh : h - nh - nkv;
    T *flat = kind == 1 ? k_out : v_out;
    if (flat) {
      dst = flat + (size_t)t * nkv * hd + (size_t)kvh * hd;
    } else {
      const int pos = tok_pos[t];
      const int page = page_table[(size_t)tok_seq[t] * P + pos / page_size];
      dst = cache + ((((size_t)page * 2 + (kind - 1)) * nkv + kvh) * page_size + pos % page_size) * hd;
    }
  }
  float *x = buf[warp];
  float ss = 0.f;
  for (int j = lane; j < hd; j += 32) {
    const float v = to_f32(src[j]);
    x[j] = v;
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  __syncwarp();
  if (w) {
    const float inv = 1.f / sqrtf(ss / (float)hd + eps);
    for (int j = lane; j < hd; j += 32) x[j] = (w[j] * x[j]) * inv;
    __syncwarp();
  }
  if (cs) {
    for (int j = lane; j < half; j += 32) {
      const float2 r = cs[j];
      const float av = x[j], bv = x[j + half];
      x[j] = av * r.x - bv * r.y;
      x[j + half] = av * r.y + bv * r.x;
    }
    __syncwarp();
  }
  for (int j = lane; j < hd; j += 32) dst[j] = from_f32<T>(x[j]);
}

template <typename T, int LPH, int E>
static void launch_qkn_fast(const void *qkv, int T_tokens, int nh, int nkv, const float *q_w, const float *k_w,
                            float eps, const float *rope_table, const int *tok_pos, const int *tok_seq,
                            const int *page_table, int P, void *cache, int page_size, void *q_out, void *k_out,
                            void *v_out, cudaStream_t stream) {
  const long long items = (long long)T_tokens * ((nh + 2 * nkv + 32 / LPH - 1) / (32 / LPH));
  const unsigned blocks = (unsigned)((items + QKN_FAST_WARPS - 1) / QKN_FAST_WARPS);
  g2b_launch(qknorm_rope_fast_kernel<T, LPH, E>, dim3(blocks), dim3(QKN_FAST_WARPS * 32), 0, stream,
             (const T *)qkv, T_tokens, nh, nkv, q_w, k_w, eps, (const float2 *)rope_table, tok_pos, tok_seq,
             page_table, P, (T *)cache, page_size, (T *)q_out, (T *)k_out, (T *)v_out);
}

extern "C" int g2b_qknorm_rope_cache(const void *qkv, int dtype, int T_tokens, int nh, int nkv,
                                     int hd, const float *q_w, const float *k_w, float eps,
                                     const float *rope_table, int rot_dim, const int *tok_pos,
                                     const int *tok_seq, const int *page_table, int P,
                                     void *cache, int page_size, void *q_out, void *k_out,
                                     void *v_out, cudaStream_t stream) {
  if (T_tokens <= 0) return 0;
  if (dtype != G2B_F32 && dtype != G2B_BF16) G2B_REFUSE("qknorm_rope_cache: unknown dtype %d", dtype);
  if (hd <= 0 || hd > QKN_MAX_HD)
    G2B_REFUSE("qknorm_rope_cache: head_dim %d outside 1..%d", hd, QKN_MAX_HD);
  if (rope_table && (rot_dim <= 0 || rot_dim > hd || (rot_dim & 1)))
    G2B_REFUSE("qknorm_rope_cache: rotary_dim %d must be even and at most head_dim %d", rot_dim, hd);
  if ((k_out == nullptr) != (v_out == nullptr))
    G2B_REFUSE("qknorm_rope_cache: k_out and v_out must be given together");
  if (nkv > 0 && !k_out && (!cache || !page_table || page_size <= 0))
    G2B_REFUSE("qknorm_rope_cache: no cache to write to");
  const int heads = nh + 2 * nkv;
  // eight elements per lane and half for prompts (many rows), four for the few rows of a decode step
  const bool wide = hd % 16 == 0 && hd >= 32 && (long long)T_tokens * heads >= 4096;
  const int epl = wide ? 8 : 4;
  const int lph = hd / (2 * epl);
  const bool aligned = (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)cache | (uintptr_t)k_out |
                         (uintptr_t)v_out | (uintptr_t)rope_table | (uintptr_t)q_w | (uintptr_t)k_w) & 15) == 0;
  const bool fast = aligned && hd % (2 * epl) == 0 && lph >= 2 && lph <= 32 && (lph & (lph - 1)) == 0 &&
                    (!rope_table || rot_dim == hd) && (long long)T_tokens * heads < (1ll << 31);
  if (fast) {
#define G2B_QKN_FAST(L)                                                                                     \
  case L:                                                                                                   \
    if (dtype == G2B_F32 && wide)                                                                           \
      launch_qkn_fast<float, L, 8>(qkv, T_tokens, nh, nkv, q_w, k_w, eps, rope_table, tok_pos, tok_seq,     \
                                   page_table, P, cache, page_size, q_out, k_out, v_out, stream);           \
    else if (dtype == G2B_F32)                                                                              \
      launch_qkn_fast<float, L, 4>(qkv, T_tokens, nh, nkv, q_w, k_w, eps, rope_table, tok_pos, tok_seq,     \
                                   page_table, P, cache, page_size, q_out, k_out, v_out, stream);           \
    else if (wide)                                                                                          \
      launch_qkn_fast<bf16, L, 8>(qkv, T_tokens, nh, nkv, q_w, k_w, eps, rope_table, tok_pos, tok_seq,      \
                                  page_table, P, cache, page_size, q_out, k_out, v_out, stream);            \
    else                                                                                                    \
      launch_qkn_fast<bf16, L, 4>(qkv, T_tokens, nh, nkv, q_w, k_w, eps, rope_table, tok_pos, tok_seq,      \
                                  page_table, P, cache, page_size, q_out, k_out, v_out, stream);            \
    break;
    switch (lph) {
      G2B_QKN_FAST(2) G2B_QKN_FAST(4) G2B_QKN_FAST(8) G2B_QKN_FAST(16) G2B_QKN_FAST(32)
    }
#undef G2B_QKN_FAST
    return g2b_check_launch("qknorm_rope_cache");
  }
  const long long items = (long long)T_tokens * heads;
  const unsigned blocks = (unsigned)((items + QKN_WARPS - 1) / QKN_WARPS);
  if (dtype == G2B_F32)
    g2b_launch(qknorm_rope_cache_kernel<float>, dim3(blocks), dim3(QKN_WARPS * 32), 0, stream,
        (const float *)qkv, T_tokens, nh, nkv, hd, q_w, k_w, eps, (const float2 *)rope_table, rot_dim,
        tok_pos, tok_seq, page_table, P, (float *)cache, page_size, (float *)q_out, (float *)k_out,
        (float *)v_out);
  else
    g2b_launch(qknorm_rope_cache_kernel<bf16>, dim3(blocks), dim3(QKN_WARPS * 32), 0, stream,
        (const bf16 *)qkv, T_tokens, nh, nkv, hd, q_w, k_w, eps, (const float2 *)rope_table, rot_dim,
        tok_pos, tok_seq, page_table, P, (bf16 *)cache, page_size, (bf16 *)q_out, (bf16 *)k_out,
        (bf16 *)v_out);
  return g2b_check_launch("qknorm_rope_cache");
}

// ---------------------------------------------------------------------------
// cache write alone: k, v [T, nkv*hd] -> the layer's pages
// ---------------------------------------------------------------------------
template <typename T>
__global__ void cache_write_kernel(const T *__restrict__ k, const T *__restrict__ v, int nkv,
                                   int hd, const int *__restrict__ tok_pos,
                                   const int *__restrict__ tok_seq,
                                   const int *__restrict__ page_table, int P,
                                   T *__restrict__ cache, int page_size) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int page = page_table[(size_t)tok_seq[t] * P + pos / page_size];
  const int n = nkv * hd;
  for (int i = threadIdx.x; i < 2 * n; i += blockDim.x) {
    const int which = i / n, r = i % n, kvh = r / hd, j = r % hd;
    const T val = (which == 0 ? k : v)[(size_t)t * n + r];
    cache[((((size_t)page * 2 + which) * nkv + kvh) * page_size + pos % page_size) * hd + j] = val;
  }
}

extern "C" int g2b_cache_write(const void *k, const void *v, int dtype, int T_tokens, int nkv,
                               int hd, const int *tok_pos, const int *tok_seq,
                               const int *page_table, int P, void *cache, int page_size,
                               cudaStream_t stream) {
  if (T_tokens <= 0) return 0;
  if (dtype == G2B_F32)
    g2b_launch(cache_write_kernel<float>, dim3(T_tokens), dim3(128), 0, stream, 
        (const float *)k, (const float *)v, nkv, hd, tok_pos, tok_seq, page_table, P,
        (float *)cache, page_size);
  else if (dtype == G2B_BF16)
    g2b_launch(cache_write_kernel<bf16>, dim3(T_tokens), dim3(128), 0, stream, 
        (const bf16 *)k, (const bf16 *)v, nkv, hd, tok_pos, tok_seq, page_table, P, (bf16 *)cache,
        page_size);
  else
    G2B_REFUSE("cache_write: unknown dtype %d", dtype);
  return g2b_check_launch("cache_write");
}

// ---------------------------------------------------------------------------
// SiLU gate on a fused gate/up projection.  Rows of the fused matrix alternate in
// blocks of `blk`: columns [2*blk*b, 2*blk*b+blk) are gate_{blk*b ..}, the next blk are
// up_{blk*b ..}; blk == I means "all gates, then all ups".
//   out[t, i] = (g / (1 + exp(-g))) * u
// ---------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T *__restrict__ gu, T *__restrict__ out, long long total,
                              int I, int blk) {
  pdl_launch();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / I;
  const int i = (int)(idx % I);
  const int b = i / blk, r = i % blk;
  const T *row = gu + (size_t)t * 2 * I;
  const float g = to_f32(row[(size_t)2 * blk * b + r]);
  const float u = to_f32(row[(size_t)2 * blk * b + blk + r]);
  out[idx] = from_f32<T>((g / (1.f + expf(-g))) * u);
}

extern "C" int g2b_swiglu(const void *gu, int dtype, int T_tokens, int I, int blk, void *out,
                          cudaStream_t stream) {
  if (T_tokens <= 0) return 0;
  if (I <= 0 || blk <= 0 || I % blk) G2B_REFUSE("swiglu: block %d does not divide width %d", blk, I);
  const long long total = (long long)T_tokens * I;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == G2B_F32)
    g2b_launch(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float *)gu, (float *)out, total, I, blk);
  else if (dtype == G2B_BF16)
    g2b_launch(swiglu_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16 *)gu, (bf16 *)out, total, I, blk);
  else
    G2B_REFUSE("swiglu: unknown dtype %d", dtype);
  return g2b_check_launch("swiglu");
}

// ---------------------------------------------------------------------------
// decode bookkeeping on the device, for steps replayed from a CUDA graph:
// positions advance by one.
// ---------------------------------------------------------------------------
__global__ void advance_positions_kernel(int *tok_pos, int n) {
  pdl_launch();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) tok_pos[i] += 1;
}

extern "C" int g2b_advance_positions(int *tok_pos, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  g2b_launch(advance_positions_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, tok_pos, n);
  return g2b_check_launch("advance_positions");
}

// Undoes the bookkeeping of one decode step that was launched ahead and is not wanted after
// all: positions go back by one and, when that step drew a random number, so do the draw
// counters of the sequences' sampling records, and the count of its recent ids when that step added one.
// (words 3 and 4 of a record: the draw counter and the count of ids in the ring of recent ids;
// the id that the step wrote stays in the ring, one place past the window)
__global__ void rewind_step_kernel(int *tok_pos, int n, int *seq_state, int words, const int *slots, int undo_draw,
                                   int undo_recent) {
  pdl_launch();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  tok_pos[i] = max(tok_pos[i] - 1, 0);          // a row of padding may have been set back to 0 since the step
  if (undo_draw) seq_state[(size_t)slots[i] * words + 3] -= 1;
  if (undo_recent) seq_state[(size_t)slots[i] * words + 4] -= 1;
}

extern "C" int g2b_rewind_step(int *tok_pos, int n, int *seq_state, int words, const int *slots, int undo_draw,
                               int undo_recent, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((undo_draw || undo_recent) && (!seq_state || !slots || words < 5))
    G2B_REFUSE("rewind_step: no sampling records to rewind");
  g2b_launch(rewind_step_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, tok_pos, n, seq_state, words, slots,
             undo_draw, undo_recent);
  return g2b_check_launch("rewind_step");
}
