// Causal grouped-query attention over the paged cache, 32-bit arithmetic, any head size
// up to 512: one warp per (token, query head).  It serves prompts and single tokens
// alike (every token carries its own position), is the attention of the float32 path,
// and the fallback of the bfloat16 path for head sizes the tensor-core kernels refuse.
//
// Formula (src/l5_model.c:518, 559-577 of AnonymoDGH/gguf2bin): kv head = head / group;
// s_t = (q . K_t) * scale for t <= pos (the loop bound is the causal mask); softmax with
// the maximum subtracted (src/l3_math.c:52-56); o = sum_t p_t V_t.  `window` > 0 keeps
// only the keys with pos - window < t <= pos.
//
// Keys are visited in chunks of 32 that start at absolute positions that are multiples
// of 32, with a running maximum and sum, so the arithmetic for a (token, head) depends
// only on its own position: not on how the tokens were cut into steps, nor on the batch.
#include "common.cuh"

G2B_DEFINE_LAST_ERROR

#define AG_MAX_HD 512
#define AG_WARPS 4

template <typename T>
__global__ void __launch_bounds__(AG_WARPS * 32)
attn_generic_kernel(const T *__restrict__ q, T *__restrict__ out, const T *__restrict__ cache,
                    const int *__restrict__ tok_pos, const int *__restrict__ tok_seq,
                    const int *__restrict__ page_table, int P, int n_tokens, int nh, int nkv,
                    int hd, int page_size, int window, float scale) {
  pdl_launch();
  pdl_wait();
  __shared__ float qs[AG_WARPS][AG_MAX_HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * AG_WARPS + warp;
  if (item >= (long long)n_tokens * nh) return;
  const int t = (int)(item / nh), h = (int)(item % nh);
  const int pos = tok_pos[t], b = tok_seq[t];
  const int kvh = h / (nh / nkv);
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;

  const T *qp = q + (size_t)t * nh * hd + (size_t)h * hd;
  for (int j = lane; j < hd; j += 32) qs[warp][j] = to_f32(qp[j]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[AG_MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < AG_MAX_HD / 32; ++i) acc[i] = 0.f;

  const size_t head_stride = (size_t)page_size * hd;              // one (page, K|V, kv head) panel
  for (int base = (lo / 32) * 32; base <= pos; base += 32) {
    const int page = page_table[(size_t)b * P + base / page_size];
    const T *kpanel = cache + (((size_t)page * 2 + 0) * nkv + kvh) * head_stride;
    const T *vpanel = cache + (((size_t)page * 2 + 1) * nkv + kvh) * head_stride;
    const int in_page = base % page_size;                         // chunk lies inside one page
    const int key = base + lane;
    const bool valid = key >= lo && key <= pos;
    float s = -INFINITY;
    if (valid) {
      const T *kr = kpanel + (size_t)(in_page + lane) * hd;
      float dot = 0.f;
      for (int j = 0; j < hd; ++j) dot = fmaf(qs[warp][j], to_f32(kr[j]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));                    // finite: key `pos` or `base` valid
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);                           // 0 on the first chunk
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < AG_MAX_HD / 32; ++i) acc[i] *= corr;
    const int n_keys = min(32, pos - base + 1);
    for (int j = 0; j < n_keys; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      if (base + j < lo) continue;
      const T *vr = vpanel + (size_t)(in_page + j) * hd;
#pragma unroll
      for (int i = 0; i < AG_MAX_HD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
      }
    }
    m = m_new;
  }
  T *op = out + (size_t)t * nh * hd + (size_t)h * hd;
  const float inv_l = 1.f / l;
#pragma unroll
  for (int i = 0; i < AG_MAX_HD / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) op[d] = from_f32<T>(acc[i] * inv_l);
  }
}

extern "C" int g2b_attn_generic(const void *q, void *out, int dtype, const void *cache,
                                const int *tok_pos, const int *tok_seq, const int *page_table,
                                int P, int n_tokens, int nh, int nkv, int hd, int page_size,
                                int window, float scale, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hd <= 0 || hd > AG_MAX_HD) G2B_REFUSE("attn_generic: head_dim %d outside 1..%d", hd, AG_MAX_HD);
  if (nkv <= 0 || nh % nkv) G2B_REFUSE("attn_generic: %d heads are not a multiple of %d kv heads", nh, nkv);
  if (page_size <= 0 || page_size % 32)
    G2B_REFUSE("attn_generic: page size %d must be a multiple of 32", page_size);
  const long long items = (long long)n_tokens * nh;
  const unsigned blocks = (unsigned)((items + AG_WARPS - 1) / AG_WARPS);
  if (dtype == G2B_F32)
    g2b_launch(attn_generic_kernel<float>, dim3(blocks), dim3(AG_WARPS * 32), 0, stream, 
        (const float *)q, (float *)out, (const float *)cache, tok_pos, tok_seq, page_table, P,
        n_tokens, nh, nkv, hd, page_size, window, scale);
  else if (dtype == G2B_BF16)
    g2b_launch(attn_generic_kernel<bf16>, dim3(blocks), dim3(AG_WARPS * 32), 0, stream, 
        (const bf16 *)q, (bf16 *)out, (const bf16 *)cache, tok_pos, tok_seq, page_table, P,
        n_tokens, nh, nkv, hd, page_size, window, scale);
  else
    G2B_REFUSE("attn_generic: unknown dtype %d", dtype);
  return g2b_check_launch("attn_generic");
}
