// Pieces shared by the one-row decode kernels (per-launch kernels and the persistent chain kernel).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace lb {
namespace {

// (d*sc, dmin*m) of sub-blocks 2t and 2t+1 from one header; `hi` = t >= 2, sh = 16 * (t & 1).
__device__ __forceinline__ void q4k_scales(const uint4 &h, bool hi, int sh, float (&dsc)[2], float (&dmn)[2]) {
  const __half2 dd = *reinterpret_cast<const __half2 *>(&h.x);
  const float2 df = __half22float2(dd);  // (d, dmin)
  // packed 6-bit fields as one byte each: sub-blocks 0..3 (lo words) or 4..7 (hi words)
  const uint32_t scw = hi ? ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u)) : (h.y & 0x3F3F3F3Fu);
  const uint32_t mnw = hi ? (((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u)) : (h.z & 0x3F3F3F3Fu);
  const uint32_t s2 = scw >> sh, m2 = mnw >> sh;
  dsc[0] = df.x * (float)(s2 & 0xFFu);
  dsc[1] = df.x * (float)((s2 >> 8) & 0xFFu);
  dmn[0] = df.y * (float)(m2 & 0xFFu);
  dmn[1] = df.y * (float)((m2 >> 8) & 0xFFu);
}

}  // namespace
}  // namespace lb
