// Counter-based Gaussian stream shared by every kernel that needs the perturbation z.
//
// z for element e of tensor t under seed s is a pure function of (s, t, e):
//   words = Philox4x32-7(counter = (e >> 3, t, stream, 0), key = (s_lo, s_hi))
//   word  = words[(e & 7) >> 1];  u = word & 0xffff for even e, word >> 16 for odd e
//   z     = T[u],  T[i] = bf16( Phi^-1((i + 0.5) / 65536) )     (65536-entry inverse-CDF table)
// so one Philox call yields the 8 normals of one 16-byte group of bf16 parameters, z is
// never stored, any sharding of a tensor (data-, tensor- or fully-sharded-parallel) sees
// the same values, and the host oracle (same table, same integers) reproduces z bit for bit.
// The table (128 KB of bf16 bit patterns) is built once on the host and staged into shared
// memory by the sweep kernel; a lookup replaces the log / sqrt / sin / cos of a Box-Muller
// transform, which made the sweep instruction-bound at half the HBM rate.  Entries are bf16
// so that two lookups merge into one bf16x2 register and theta + c z runs as one packed
// fma.rn.bf16x2 per pair of parameters (perturb8_packed): no unpack, convert or repack
// instructions, a single rounding.  The reference instead re-seeds torch's generator and
// materialises z per tensor (large_models/trainer.py:1438-1444, :1603-1608).
#pragma once
#include <stdint.h>
#ifdef __CUDACC__
#include <cuda_bf16.h>
#endif

namespace dz {

constexpr uint32_t PHILOX_M0 = 0xD2511F53u;
constexpr uint32_t PHILOX_M1 = 0xCD9E8D57u;
constexpr uint32_t PHILOX_W0 = 0x9E3779B9u;
constexpr uint32_t PHILOX_W1 = 0xBB67AE85u;

struct Philox4 {
  uint32_t x, y, z, w;
};

template <int ROUNDS = 10>
__host__ __device__ __forceinline__ Philox4 philox4x32(uint32_t c0, uint32_t c1, uint32_t c2,
                                                       uint32_t c3, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
    // one widening 32x32->64 multiply per product, both halves used
    const uint64_t p0 = static_cast<uint64_t>(PHILOX_M0) * c0;
    const uint64_t p1 = static_cast<uint64_t>(PHILOX_M1) * c2;
    const uint32_t hi0 = static_cast<uint32_t>(p0 >> 32), lo0 = static_cast<uint32_t>(p0);
    const uint32_t hi1 = static_cast<uint32_t>(p1 >> 32), lo1 = static_cast<uint32_t>(p1);
    uint32_t n0 = hi1 ^ c1 ^ k0;
    uint32_t n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += PHILOX_W0;
    k1 += PHILOX_W1;
  }
  return Philox4{c0, c1, c2, c3};
}

#ifdef __CUDACC__
constexpr int GAUSS_TABLE_SIZE = 65536;
// Rounds of the z stream: Philox4x32 is Crush-resistant from 7 rounds (Salmon et al., SC'11; 10 is the
// library default) and the sweep spends a third of its time in them.  Must equal Z_PHILOX_ROUNDS of
// ops/philox.py (the host oracle).  Other streams (gamma draws, stochastic rounding, sampling) keep 10.
constexpr int Z_PHILOX_ROUNDS = 7;

// The Philox words of group `grp` (= element index >> 3) of tensor `tid`.
__device__ __forceinline__ Philox4 z_words(uint64_t seed, uint32_t tid, uint32_t grp, uint32_t stream) {
  return philox4x32<Z_PHILOX_ROUNDS>(grp, tid, stream, 0u, static_cast<uint32_t>(seed),
                                     static_cast<uint32_t>(seed >> 32));
}

// Table entry for a 16-bit index held in the low / high half of `w`, as raw bf16 bits.
__device__ __forceinline__ uint32_t gauss_bits_lo(const uint16_t* tab, uint32_t w) {
  return *reinterpret_cast<const uint16_t*>(reinterpret_cast<const char*>(tab) + ((w & 0xffffu) << 1));
}
__device__ __forceinline__ uint32_t gauss_bits_hi(const uint16_t* tab, uint32_t w) {
  return *reinterpret_cast<const uint16_t*>(reinterpret_cast<const char*>(tab) + ((w >> 15) & 0x1fffeu));
}

// The 8 normals of a group as fp32; `tab` may point to shared or global memory.
__device__ __forceinline__ void gauss8(const uint16_t* tab, uint64_t seed, uint32_t tid, uint32_t grp,
                                       uint32_t stream, float z[8]) {
  const Philox4 p = z_words(seed, tid, grp, stream);
  const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    z[2 * j] = __uint_as_float(gauss_bits_lo(tab, w[j]) << 16);
    z[2 * j + 1] = __uint_as_float(gauss_bits_hi(tab, w[j]) << 16);
  }
}

// The 8 normals of a group as four bf16x2 registers (element 2j in the low half of word j).
__device__ __forceinline__ void gauss8_packed(const uint16_t* tab, uint64_t seed, uint32_t tid,
                                              uint32_t grp, uint32_t stream, uint32_t zp[4]) {
  const Philox4 p = z_words(seed, tid, grp, stream);
  const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
  for (int j = 0; j < 4; ++j)
    zp[j] = __byte_perm(gauss_bits_lo(tab, w[j]), gauss_bits_hi(tab, w[j]), 0x5410);
}

// theta + c z for one 16-byte group of bf16 parameters: four fma.rn.bf16x2, each an exact
// product and sum rounded once to bf16.  `c2` holds the coefficient (rounded to bf16) in both halves.
__device__ __forceinline__ uint4 perturb8_packed(const uint16_t* tab, uint64_t seed, uint32_t tid,
                                                 uint32_t grp, uint32_t c2, uint4 raw) {
  uint32_t zp[4];
  gauss8_packed(tab, seed, tid, grp, 0u, zp);
  uint32_t v[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; ++j)
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(v[j]) : "r"(c2), "r"(zp[j]), "r"(v[j]));
  return make_uint4(v[0], v[1], v[2], v[3]);
}

// A coefficient rounded to bf16 and replicated into both halves of a bf16x2 register.
__device__ __forceinline__ uint32_t bf16x2_splat(float c) {
  __nv_bfloat162 v = __float2bfloat162_rn(c);
  return *reinterpret_cast<uint32_t*>(&v);
}
#endif

}  // namespace dz
