// Random weights made on the device: a counter-based normal generator whose value at an
// element depends on (seed, index of the tensor in the model's list, index of the element)
// and on nothing else, so a tensor can be filled in place, in any order, on any device,
// and the CPU (weights/random_init.py) gets the same bits.
//
// The reference makes its synthetic model in-process too (src/l5_model.c:634-680 of
// AnonymoDGH/gguf2bin), but fills the matrices with zeros, which hides every fault; here
// matrices are N(0, std) and scale vectors 1 + N(0, scale_std).
//
// Definition (every arithmetic step is ONE IEEE binary32 operation, rounded to nearest even,
// never contracted into a fused multiply-add; that is what makes CPU and GPU agree):
//   block = element / 4;  lane = element % 4
//   (w0..w3) = Philox4x32-10(counter = (block lo, block hi, tensor index, 0x6e6f726d),
//                            key = (seed lo, seed hi))
//   lanes 0,1 use (a, b) = (w0, w1); lanes 2,3 use (w2, w3)            [Box-Muller]
//   k1 = (a >> 8) + 1 in [1, 2^24], u1 = k1 / 2^24;  k2 = b >> 8 in [0, 2^24)
//   ln u1 = (e - 24) * ln2 + ln m,  k1 = m * 2^e with m in [1, 2);
//           ln m = 2 s (1 + s^2/3 + s^4/5 + ... + s^12/13),  s = (m - 1) / (m + 1)   (Horner in s^2)
//   r = sqrt(-2 ln u1)
//   quadrant q = k2 >> 22, x = ((k2 & (2^22 - 1)) / 2^22) * (pi/2)
//   sin x, cos x by their Taylor polynomials to x^11 and x^12 (Horner in x^2), turned by q
//   z = r * cos (even lane) or r * sin (odd lane)
//   value = std * z   (matrix)   or   1 + std * z   (scale vector)
//   stored as binary32, or rounded to bfloat16 (nearest even)
#include "common.cuh"

G2B_DEFINE_LAST_ERROR

__device__ __forceinline__ void philox_normal_block(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                                    uint32_t k0, uint32_t k1, uint32_t w[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  w[0] = c0; w[1] = c1; w[2] = c2; w[3] = c3;
}

// Two standard normals from two 32-bit words; see the definition above.
__device__ __forceinline__ void box_muller_exact(uint32_t a, uint32_t b, float &z_cos, float &z_sin) {
  const uint32_t k1 = (a >> 8) + 1u;                       // 1 .. 2^24
  const int e = 31 - __clz((int)k1);                       // k1 = m * 2^e
  const float m = __fmul_rn((float)k1, __int_as_float((127 - e) << 23));      // exact
  const float s = __fdiv_rn(__fadd_rn(m, -1.0f), __fadd_rn(m, 1.0f));
  const float s2 = __fmul_rn(s, s);
  float p = 0x1.3b13b2p-4f;                                // 1/13
  p = __fadd_rn(__fmul_rn(p, s2), 0x1.745d18p-4f);         // 1/11
  p = __fadd_rn(__fmul_rn(p, s2), 0x1.c71c72p-4f);         // 1/9
  p = __fadd_rn(__fmul_rn(p, s2), 0x1.24924ap-3f);         // 1/7
  p = __fadd_rn(__fmul_rn(p, s2), 0x1.99999ap-3f);         // 1/5
  p = __fadd_rn(__fmul_rn(p, s2), 0x1.555556p-2f);         // 1/3
  p = __fadd_rn(__fmul_rn(p, s2), 1.0f);
  const float ln_m = __fmul_rn(__fmul_rn(2.0f, s), p);
  const float ln_u = __fadd_rn(__fmul_rn((float)(e - 24), 0x1.62e430p-1f), ln_m);   // ln 2
  const float r = __fsqrt_rn(__fmul_rn(-2.0f, ln_u));

  const uint32_t k2 = b >> 8;
  const uint32_t q = k2 >> 22;
  const float f = __fmul_rn((float)(k2 & 0x3fffffu), 0x1p-22f);                 // exact
  const float x = __fmul_rn(f, 0x1.921fb6p+0f);                                 // pi/2
  const float x2 = __fmul_rn(x, x);
  float ps = -0x1.ae6456p-26f;                             // -1/11!
  ps = __fadd_rn(__fmul_rn(ps, x2), 0x1.71de3ap-19f);      //  1/9!
  ps = __fadd_rn(__fmul_rn(ps, x2), -0x1.a01a02p-13f);     // -1/7!
  ps = __fadd_rn(__fmul_rn(ps, x2), 0x1.111112p-7f);       //  1/5!
  ps = __fadd_rn(__fmul_rn(ps, x2), -0x1.555556p-3f);      // -1/3!
  ps = __fadd_rn(__fmul_rn(ps, x2), 1.0f);
  const float sn = __fmul_rn(x, ps);
  float pc = 0x1.1eed8ep-29f;                              //  1/12!
  pc = __fadd_rn(__fmul_rn(pc, x2), -0x1.27e4fcp-22f);     // -1/10!
  pc = __fadd_rn(__fmul_rn(pc, x2), 0x1.a01a02p-16f);      //  1/8!
  pc = __fadd_rn(__fmul_rn(pc, x2), -0x1.6c16c2p-10f);     // -1/6!
  pc = __fadd_rn(__fmul_rn(pc, x2), 0x1.555556p-5f);       //  1/4!
  pc = __fadd_rn(__fmul_rn(pc, x2), -0.5f);
  const float cs = __fadd_rn(__fmul_rn(pc, x2), 1.0f);
  // turn by the quadrant: angle = q * pi/2 + x
  const float c = q == 0 ? cs : q == 1 ? -sn : q == 2 ? -cs : sn;
  const float sq = q == 0 ? sn : q == 1 ? cs : q == 2 ? -sn : -cs;
  z_cos = __fmul_rn(r, c);
  z_sin = __fmul_rn(r, sq);
}

template <typename T>
__global__ void philox_normal_kernel(T *__restrict__ out, long long n, uint32_t seed_lo,
                                     uint32_t seed_hi, uint32_t tensor_index, int scale_vector,
                                     float std) {
  const long long n_blocks = (n + 3) / 4;
  for (long long blk = (long long)blockIdx.x * blockDim.x + threadIdx.x; blk < n_blocks;
       blk += (long long)gridDim.x * blockDim.x) {
    uint32_t w[4];
    philox_normal_block((uint32_t)(blk & 0xffffffffll), (uint32_t)(blk >> 32), tensor_index,
                        0x6e6f726du, seed_lo, seed_hi, w);
    float z[4];
    box_muller_exact(w[0], w[1], z[0], z[1]);
    box_muller_exact(w[2], w[3], z[2], z[3]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const long long at = blk * 4 + i;
      if (at < n) {
        float v = __fmul_rn(std, z[i]);
        if (scale_vector) v = __fadd_rn(1.0f, v);
        out[at] = from_f32<T>(v);
      }
    }
  }
}

// Fills out[0..n) in place.  kind 0: N(0, std); kind 1: 1 + N(0, std).
extern "C" int g2b_philox_normal(void *out, int dtype, long long n, unsigned long long seed,
                                 unsigned int tensor_index, int kind, float std, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (kind != 0 && kind != 1) G2B_REFUSE("philox_normal: kind must be 0 (matrix) or 1 (scale vector), got %d", kind);
  if (!(std >= 0.f)) G2B_REFUSE("philox_normal: the standard deviation must not be negative, got %g", std);
  const long long n_blocks = (n + 3) / 4;
  const int threads = 256;
  long long grid = (n_blocks + threads - 1) / threads;
  if (grid > 148ll * 32) grid = 148ll * 32;
  const uint32_t lo = (uint32_t)(seed & 0xffffffffull), hi = (uint32_t)(seed >> 32);
  if (dtype == G2B_F32)
    philox_normal_kernel<float><<<(unsigned)grid, threads, 0, stream>>>((float *)out, n, lo, hi, tensor_index, kind, std);
  else if (dtype == G2B_BF16)
    philox_normal_kernel<bf16><<<(unsigned)grid, threads, 0, stream>>>((bf16 *)out, n, lo, hi, tensor_index, kind, std);
  else
    G2B_REFUSE("philox_normal: unknown dtype %d", dtype);
  return g2b_check_launch("philox_normal");
}
