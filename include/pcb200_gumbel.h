/* pcb200_gumbel.h — the Gumbel-max key, shared bit for bit by host and device.
 *
 * Hard sampling picks argmax_j (logp_j + g(u_j)) with
 *     g(u) = -log(-log(u * (1.0 - 1e-6) + 1e-6))
 * which is the noise expression of VariationalJuice.jl/src/queries/sample.jl:45 evaluated
 * in Float64 (Julia promotes through the Float64 literals).  A sample is only reproducible
 * across CPU and GPU if both sides produce the same 64-bit key, and the C library's log and
 * CUDA's log may differ in the last place.  So the logarithm below is built from IEEE
 * add / multiply / divide / fma only, each rounded to nearest and never re-associated or
 * contracted: on the device through the __d*_rn intrinsics, on the host through plain
 * operators in a translation unit compiled with -ffp-contract=off.
 *
 * log(x), x = 2^e * m, m in [sqrt(1/2), sqrt(2)):  with s = (m-1)/(m+1),
 *     log(m) = 2 atanh(s) = 2 s (1 + s^2/3 + s^4/5 + ... + s^22/23),   |s| <= 0.1716
 * (the truncation error is below 2^-58 relative).
 */
#ifndef PCB200_GUMBEL_H
#define PCB200_GUMBEL_H

#include <stdint.h>
#include <string.h>

#if defined(__CUDA_ARCH__)
#define PCB_HD __host__ __device__ __forceinline__
#define PCB_MUL(a, b) __dmul_rn((a), (b))
#define PCB_ADD(a, b) __dadd_rn((a), (b))
#define PCB_DIV(a, b) __ddiv_rn((a), (b))
#define PCB_FMA(a, b, c) __fma_rn((a), (b), (c))
#else
#include <math.h>
#if defined(__CUDACC__)
#define PCB_HD __host__ __device__ __forceinline__
#else
#define PCB_HD static inline
#endif
#define PCB_MUL(a, b) ((a) * (b))
#define PCB_ADD(a, b) ((a) + (b))
#define PCB_DIV(a, b) ((a) / (b))
#define PCB_FMA(a, b, c) fma((a), (b), (c))
#endif

PCB_HD double pcb_bits_to_double(uint64_t b) {
#if defined(__CUDA_ARCH__)
  return __longlong_as_double((long long)b);
#else
  double d;
  memcpy(&d, &b, sizeof d);
  return d;
#endif
}
PCB_HD uint64_t pcb_double_to_bits(double d) {
#if defined(__CUDA_ARCH__)
  return (uint64_t)__double_as_longlong(d);
#else
  uint64_t b;
  memcpy(&b, &d, sizeof b);
  return b;
#endif
}

/* natural log of a positive, finite, normal double */
PCB_HD double pcb_log(double x) {
  uint64_t bits = pcb_double_to_bits(x);
  int64_t e = (int64_t)((bits >> 52) & 0x7ffull) - 1023;
  double m = pcb_bits_to_double((bits & 0x000fffffffffffffull) | 0x3ff0000000000000ull);
  if (m > 1.4142135623730951) {
    m = PCB_MUL(m, 0.5);
    e += 1;
  }
  double f = PCB_ADD(m, -1.0);
  double s = PCB_DIV(f, PCB_ADD(m, 1.0));
  double z = PCB_MUL(s, s);
  double p = 1.0 / 23.0;
  p = PCB_FMA(p, z, 1.0 / 21.0);
  p = PCB_FMA(p, z, 1.0 / 19.0);
  p = PCB_FMA(p, z, 1.0 / 17.0);
  p = PCB_FMA(p, z, 1.0 / 15.0);
  p = PCB_FMA(p, z, 1.0 / 13.0);
  p = PCB_FMA(p, z, 1.0 / 11.0);
  p = PCB_FMA(p, z, 1.0 / 9.0);
  p = PCB_FMA(p, z, 1.0 / 7.0);
  p = PCB_FMA(p, z, 1.0 / 5.0);
  p = PCB_FMA(p, z, 1.0 / 3.0);
  double two_s = PCB_ADD(s, s);
  double lm = PCB_FMA(PCB_MUL(two_s, z), p, two_s);
  return PCB_FMA((double)e, 0.6931471805599453, lm);
}

/* logp + g(u), u uniform in [0, 1) */
PCB_HD double pcb_gumbel_key(float logp, float u) {
  double x = PCB_ADD(PCB_MUL((double)u, 1.0 - 1e-6), 1e-6);
  double inner = -pcb_log(x);       /* in (0, 13.9] */
  double g = -pcb_log(inner);
  return PCB_ADD((double)logp, g);
}

/* 64-bit mixer (splitmix64 finaliser) used for scope signatures of sum regions */
PCB_HD uint64_t pcb_scope_mix(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

#endif /* PCB200_GUMBEL_H */
