// Walk specification shared by the device kernels and the host-side graph
// generator: the counter-based random stream, the exponential key and the
// strip geometry.  Everything here is integer arithmetic or correctly rounded
// fp32 (+, *, /, fma), so host and device produce identical bits.
#pragma once
#include <stdint.h>
#include <math.h>

#if defined(__CUDACC__)
#define FW_HD __host__ __device__ __forceinline__
#else
#define FW_HD inline
#endif

namespace fw {

// What a Philox block is used for (upper 4 bits of counter word 1).
constexpr uint32_t kPurposeScan = 0u;  // keys of the row scan
constexpr uint32_t kPurposeStop = 1u;  // PPR stop test after a step

// A row [b,e) of the CSR is addressed in aligned quads of 4 edges (16 bytes):
// quad q covers absolute edges 4*(q0+q) .. +3 with q0 = b>>2.  A sub-block is
// 128 consecutive quads (2 KB, what a warp loads with four 16-byte accesses per
// lane); a supergroup is four sub-blocks (512 quads, 8 KB).  Strip (s,l) holds
// the 16 quads s*512 + j*32 + l, j = 0..15 -- everything lane l touches when a
// warp sweeps supergroup s.  Its total bias is summed in a fixed order: per
// quad (w0+w1)+(w2+w3), per sub-block (S0+S1)+(S2+S3), then (A0+A1)+(A2+A3).
// Strip (s,l) has id B = s*32 + l; its key uses word s%3 of the scan block
// with counter word 0 = (s/3)*32 + l (one Philox block serves three
// supergroups of a lane); word 3 of that block is the uniform for the pick
// inside the winning strip.
constexpr int kQuadsPerSub = 128;
constexpr int kSubsPerSuper = 4;
constexpr int kQuadsPerSuper = kQuadsPerSub * kSubsPerSuper;

struct Philox4 { uint32_t x, y, z, w; };

// Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy
// as 1, 2, 3", SC'11).  Counter (c0..c3), key (k0,k1).
FW_HD Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                            uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    c1 = (uint32_t)p1;
    c3 = (uint32_t)p0;
    c0 = n0;
    c2 = n2;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return Philox4{c0, c1, c2, c3};
}

// The same function with the ten round keys formed ahead of time: rk[2r] = k0 + r * 0x9E3779B9,
// rk[2r+1] = k1 + r * 0xBB67AE85 (mod 2^32).  A kernel that keeps them among its arguments
// reads each straight from the constant bank and saves the key schedule of every call.
FW_HD void philox_round_keys(uint32_t k0, uint32_t k1, uint32_t rk[20]) {
  for (int r = 0; r < 10; ++r) {
    rk[2 * r] = k0;
    rk[2 * r + 1] = k1;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

FW_HD Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, const uint32_t (&rk)[20]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ rk[2 * r];
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ rk[2 * r + 1];
    c1 = (uint32_t)p1;
    c3 = (uint32_t)p0;
    c0 = n0;
    c2 = n2;
  }
  return Philox4{c0, c1, c2, c3};
}

FW_HD int clz32(uint32_t x) {
#if defined(__CUDA_ARCH__)
  return __clz((int)x);
#else
  return x ? __builtin_clz(x) : 32;
#endif
}

// 32 random bits -> exponential variate in log2 units, E = g + f(m), where g
// is the number of leading zero bits (geometric, P(g) = 2^-(g+1)), m in (0,1]
// is the fraction formed by the bits after the leading one, and
// f(m) = -log2(1 - m/2) evaluated as m*P(m) with a fixed degree-5 polynomial
// (relative error < 7e-6).  The smallest keys -- the ones that win in rows of
// 10^5..10^6 neighbours -- keep full fp32 relative precision.
FW_HD float exp_key(uint32_t x) {
  const int g = clz32(x);
  const uint32_t t = x << (g & 31);
  const uint32_t mb = t << 1;
  const float m = fmaf((float)mb, 0x1p-32f, 0x1p-33f);
  float p = 0x1.3897a4p-6f;
  p = fmaf(p, m, -0x1.cb946cp-7f);
  p = fmaf(p, m, 0x1.29f26p-5f);
  p = fmaf(p, m, 0x1.cf6494p-5f);
  p = fmaf(p, m, 0x1.71fdcap-3f);
  p = fmaf(p, m, 0x1.7153dap-1f);
  return fmaf(p, m, (float)g);
}

// PPR: stop after a step iff the 32-bit draw is below this threshold.
inline uint32_t tp_threshold(double tp) {
  const double t = tp * 4294967296.0;
  if (!(t > 0.0)) return 0u;
  if (t >= 4294967295.0) return 0xFFFFFFFFu;
  return (uint32_t)t;
}

}  // namespace fw
