// In-register dequantisation of the absmax-u8 weight layout
// (Q[n,k] u8 row-major, S[n,k/bs] fp16; adrastea_kernels/cpp/quantize.cu:3-56).
//
// Target value, bit-exact:  w = fp16((float(q) - zero) * float(s))
// (matmul_nt_wmma_16x128x256_fp16u8.cu:5-7).  With the reference's constant
// zero 127.5 the fp32 product is exact (8-bit x 11-bit significands), so the
// only rounding is the final one to fp16.  That lets the fast path work on
// packed halves:
//     h  = 0x6400 | q            (fp16 value 1024 + q, exact)
//     t  = h - 1152              (q - 128, exact)
//     w  = fma(t, s, s/2)        (one rounding of (q - 127.5) * s)
// which is exact whenever s/2 is exact in fp16, i.e. for every scale with a
// biased exponent >= 2 (|s| >= 2^-13); other scales (and the zero-point
// extension) take the fp32 path, two elements per conversion.
#pragma once
#include "common.cuh"

namespace adr {

struct ScalePair {
  __half2 s2;    // (s, s)
  __half2 hs2;   // (s/2, s/2)
  float sf;      // float(s)
  float zf;      // zero point as float (127.5 unless zeros are given)
  bool fast;     // packed-half path is exact for this scale
};

__device__ __forceinline__ ScalePair make_scale(__half s, bool has_zero, __half z) {
  ScalePair p;
  unsigned short bits = __half_as_ushort(s) & 0x7FFFu;
  p.fast = !has_zero && bits >= 0x0800u && bits < 0x7C00u;
  p.s2 = __half2half2(s);
  p.hs2 = __hmul2(p.s2, __float2half2_rn(0.5f));
  p.sf = __half2float(s);
  p.zf = has_zero ? __half2float(z) : 127.5f;
  return p;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

__device__ __forceinline__ __half2 u32_as_half2(uint32_t v) {
  return *reinterpret_cast<__half2*>(&v);
}
__device__ __forceinline__ uint32_t half2_as_u32(__half2 v) {
  return *reinterpret_cast<uint32_t*>(&v);
}

// Dequantise the four bytes of `word` into two packed pairs:
// lo = (w(byte0), w(byte1)), hi = (w(byte2), w(byte3)).
__device__ __forceinline__ void dequant4(uint32_t word, const ScalePair& sp, __half2& lo,
                                         __half2& hi) {
  // (0x6400 | byte) for bytes (0,1) and (2,3)
  uint32_t m01 = prmt(word, 0x64646464u, 0x4140u);
  uint32_t m23 = prmt(word, 0x64646464u, 0x4342u);
  if (sp.fast) {
    const __half2 k1152 = u32_as_half2(0x64806480u);
    lo = __hfma2(__hsub2(u32_as_half2(m01), k1152), sp.s2, sp.hs2);
    hi = __hfma2(__hsub2(u32_as_half2(m23), k1152), sp.s2, sp.hs2);
  } else {
    const __half2 k1024 = u32_as_half2(0x64006400u);
    float2 q01 = __half22float2(__hsub2(u32_as_half2(m01), k1024));
    float2 q23 = __half22float2(__hsub2(u32_as_half2(m23), k1024));
    lo = __floats2half2_rn((q01.x - sp.zf) * sp.sf, (q01.y - sp.zf) * sp.sf);
    hi = __floats2half2_rn((q23.x - sp.zf) * sp.sf, (q23.y - sp.zf) * sp.sf);
  }
}

__device__ __forceinline__ uint4 ldg_nc_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

}  // namespace adr
