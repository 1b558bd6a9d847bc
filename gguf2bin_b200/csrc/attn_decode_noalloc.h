/* Decode attention for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in AnonymoDGH/gguf2bin (the reference is a CPU
 * program and has neither device memory nor scratch buffers); it exists for users of THIS
 * library.
 *
 * Who needs it.  The ordinary entry point, g2b_attn_decode(), takes two scratch buffers
 * (partial outputs and softmax statistics of the key chunks) that its caller allocates.
 * Some callers have no way to do that: a plugin running inside a host process whose
 * device memory is owned entirely by that host's allocator (an inference server that
 * reserved the whole GPU at start-up and forbids its plugins to call cudaMalloc), or a
 * control loop with a latency bound that cannot afford the device-wide synchronisation a
 * cudaMalloc or cudaFree may imply.  For them the scratch lives in a fixed array inside
 * the shared object.
 *
 * What it does.  Same arithmetic and same kernels as g2b_attn_decode(); the scratch is a
 * file-scope `static __device__ __align__(256)` array of G2B_NOALLOC_SCRATCH_BYTES
 * (16 MiB).  Every GPU on which this shared object is used holds those 16 MiB from the
 * moment its code is loaded there until the process exits.  The call allocates nothing:
 * no cudaMalloc, cudaFree or allocating library routine, torch's included.
 *
 * Limits.  With C = g2b_attn_decode_chunk_keys() (the keys one thread block takes: 256 in
 * the object as shipped, 128 in a build with -DATTN_DECODE_PAGES=2),
 * T * n_heads * ceil(max_kv_len / C) * (head_dim + 2) * 4 bytes must not exceed
 * G2B_NOALLOC_SCRATCH_BYTES.  For 16 heads of 128 and C = 256 that is 8 tokens at up to
 * 64,512 keys, or 64 tokens at up to 7,936 keys.  Larger requests are refused with a
 * message naming the limit, and nothing is launched.
 *
 * What the caller guarantees (neither entry point can check it, the positions being on
 * the device): every tok_pos[t] < max_kv_len <= P * 64.  A position at or beyond
 * max_kv_len would make the merge pass read partial results of a neighbouring head.
 * And only if the caller has switched programmatic dependent launch on (g2b_set_pdl(1);
 * it is off in a freshly loaded object): kernels of the caller that change tok_pos while
 * this one may already have started let a position grow, or shrink by at most one.
 *
 * First call.  The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current) and sets the kernel's shared-memory
 * attribute for that device; make that first call during set-up, before any stream
 * capture begins on that device.  Later calls on that device only launch.
 *
 * Sharing.  All calls in the process share the one array per device, and it keeps the
 * last call's contents.  Nothing in it has to start at zero: every partial that the
 * combine pass reads is written earlier in the same call.  Two calls that overlap on the
 * GPU (different streams, or different threads on one device) race on the array; issue
 * them on one stream or order them with events.
 *
 * Returns 0 on success; otherwise non-zero, and g2b_last_error() of the same shared
 * object returns the reason.  Arguments are those of g2b_attn_decode() without the two
 * scratch pointers: q, out [T, n_heads*head_dim] bfloat16; cache [pages][2][n_kv_heads]
 * [64][head_dim] bfloat16 of one layer; tok_pos, tok_seq [T] int32; page_table
 * [sequences, P] int32; all on the current device.
 */
#ifndef G2B_ATTN_DECODE_NOALLOC_H
#define G2B_ATTN_DECODE_NOALLOC_H

#include <cuda_runtime.h>

#define G2B_NOALLOC_SCRATCH_BYTES (16u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

int g2b_attn_decode_noalloc(const void *q, void *out, const void *cache, const int *tok_pos,
                            const int *tok_seq, const int *page_table, int P, int T, int n_heads,
                            int n_kv_heads, int head_dim, int page_size, int window, float scale,
                            int max_kv_len, cudaStream_t stream);

/* The limit above, for callers that want to check before they call. */
unsigned long long g2b_attn_decode_noalloc_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
#endif
