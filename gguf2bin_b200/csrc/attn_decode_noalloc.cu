// Allocation-free variant of the decode attention entry point: see attn_decode_noalloc.h
// for who needs it, its limits and its rules.  It has no counterpart in the reference.
//
// The kernels and the ordinary launcher are compiled into this object from attn_decode.cu
// unchanged; the only additions are the scratch array and the entry point below.
#include "attn_decode.cu"
#include "attn_decode_noalloc.h"

#include <mutex>

// The scratch of every call on a device.  In HOST code this name is only a stand-in for
// the device array: its device address comes from cudaGetSymbolAddress, below.
static __device__ __align__(256) float g2b_noalloc_scratch[G2B_NOALLOC_SCRATCH_BYTES / sizeof(float)];

constexpr int G2B_NOALLOC_MAX_DEVICES = 64;
static float *g2b_noalloc_ptr[G2B_NOALLOC_MAX_DEVICES] = {};
static std::mutex g2b_noalloc_mutex;

extern "C" unsigned long long g2b_attn_decode_noalloc_scratch_bytes(void) {
  return G2B_NOALLOC_SCRATCH_BYTES;
}

extern "C" int g2b_attn_decode_noalloc(const void *q, void *out, const void *cache,
                                       const int *tok_pos, const int *tok_seq,
                                       const int *page_table, int P, int T, int n_heads,
                                       int n_kv_heads, int head_dim, int page_size, int window,
                                       float scale, int max_kv_len, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_heads <= 0 || max_kv_len <= 0) G2B_REFUSE("attn_decode_noalloc: bad sizes");
  const long long n_chunks = ((long long)max_kv_len + CHUNK_KEYS - 1) / CHUNK_KEYS;
  const long long slots = (long long)T * n_heads * n_chunks;
  const long long need = slots * (HD + 2) * (long long)sizeof(float);
  if (need > (long long)G2B_NOALLOC_SCRATCH_BYTES)
    G2B_REFUSE("attn_decode_noalloc: %d tokens x %d heads x %lld key chunks need %lld bytes of "
               "scratch; the built-in array holds %u (use g2b_attn_decode with your own scratch)",
               T, n_heads, n_chunks, need, G2B_NOALLOC_SCRATCH_BYTES);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) G2B_REFUSE("attn_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= G2B_NOALLOC_MAX_DEVICES)
    G2B_REFUSE("attn_decode_noalloc: device %d outside 0..%d", dev, G2B_NOALLOC_MAX_DEVICES - 1);
  float *scratch;
  {
    std::lock_guard<std::mutex> lock(g2b_noalloc_mutex);
    if (!g2b_noalloc_ptr[dev]) {          // set-up, once per device, with that device current
      float *p = nullptr;
      e = cudaGetSymbolAddress((void **)&p, g2b_noalloc_scratch);
      if (e != cudaSuccess || !p)
        G2B_REFUSE("attn_decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      g2b_noalloc_ptr[dev] = p;
    }
    scratch = g2b_noalloc_ptr[dev];
  }
  float *part_o = scratch;                                    // slots * HD floats
  float *part_ml = scratch + (size_t)slots * HD;              // slots * 2 floats (8-byte aligned)
  return g2b_attn_decode(q, out, cache, tok_pos, tok_seq, page_table, P, T, n_heads, n_kv_heads,
                         head_dim, page_size, window, scale, max_kv_len, part_o, part_ml, stream);
}
