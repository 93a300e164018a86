// Counter-based Gaussian stream shared by every kernel that needs the perturbation z.
//
// z for element e of tensor t under seed s is a pure function of (s, t, e):
//   words = Philox4x32-7(counter = (e >> 3, t, stream, 0), key = (s_lo, s_hi))
//   word  = words[(e & 7) >> 1];  u = word & 0xffff for even e, word >> 16 for odd e
//   i = u & 1023 (quantile bin), k = u >> 10 (position inside the bin, 0..63)
//   z = bf16( a'_i + b_i * m_k ),  m_k = 1 + (2k + 1) / 128        (one fused multiply-add)
// i.e. the inverse normal CDF, piecewise linear over 1024 equal-probability bins: (a'_i, b_i) is
// the line with the mean and variance of the 64 quantiles Phi^-1((i + (k + 0.5)/64) / 1024) of bin i,
// shifted so that m_k can be built from the index bits alone (0x3F80 | 2k+1 is the bf16 1 + (2k+1)/128).
// One Philox call yields the 8 normals of one 16-byte group of bf16 parameters, z is never stored,
// any sharding of a tensor (data-, tensor- or fully-sharded-parallel) sees the same values, and the
// host oracle (same table, same integers, same single rounding) reproduces z bit for bit.
//
// Why this shape: a sweep at HBM rate needs about 8 normals per clock per SM.  Box-Muller
// (log / sqrt / sin / cos) was bound by the special-function unit at half the HBM rate; a
// 65536-entry inverse-CDF table in shared memory was bound by bank conflicts (32 random addresses
// per warp serialise into ~3.5 wavefronts per load).  The 1024 (a', b) pairs are 4 bytes each and
// are replicated 32 times in shared memory (128 KB) so that lane l always reads bank l: every
// lookup is one conflict-free wavefront.  The pairs stay bf16, two lookups are re-paired with
// byte permutes, and both z = b m + a' and theta + c z run as packed fma.rn.bf16x2 (exact product
// and sum, one rounding each).  The reference instead re-seeds torch's generator and materialises
// z per tensor (large_models/trainer.py:1438-1444, :1603-1608).
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
constexpr int GAUSS_BINS = 1024;                   // (a', b) pairs: low half a', high half b, both bf16
constexpr int GAUSS_SMEM_BYTES = GAUSS_BINS * 128;  // replicated per lane (bank) in shared memory
// Rounds of the z stream: Philox4x32 is Crush-resistant from 7 rounds (Salmon et al., SC'11; 10 is the
// library default) and the sweep spends a third of its instructions in them.  Must equal Z_PHILOX_ROUNDS
// of ops/philox.py (the host oracle); the stochastic-rounding stream of the update uses the same count.
// Other streams (gamma draws, sampling) keep 10.
constexpr int Z_PHILOX_ROUNDS = 7;

// The Philox words of group `grp` (= element index >> 3) of tensor `tid`.
__device__ __forceinline__ Philox4 z_words(uint64_t seed, uint32_t tid, uint32_t grp, uint32_t stream) {
  return philox4x32<Z_PHILOX_ROUNDS>(grp, tid, stream, 0u, static_cast<uint32_t>(seed),
                                     static_cast<uint32_t>(seed >> 32));
}

// Copy the 1024 pairs from global memory into the lane-replicated shared-memory layout
// (entry i, lane l at byte i * 128 + l * 4).  All threads of the CTA call it; sync afterwards.
__device__ __forceinline__ void gauss_table_to_smem(void* smem_tab, const uint32_t* gtab, int tid, int nthreads) {
  uint4* dst = reinterpret_cast<uint4*>(smem_tab);
  for (int i = tid; i < GAUSS_BINS * 8; i += nthreads) {
    const uint32_t e = __ldg(gtab + (i >> 3));
    dst[i] = make_uint4(e, e, e, e);
  }
}

// A table seen by one thread: `base` points at this thread's copy of entry 0, entries are
// (1 << SHIFT) bytes apart.  SHIFT 7: the lane-replicated shared-memory copy (base = table + 4 * lane);
// SHIFT 2: the plain 1024-word table in global memory.
template <int SHIFT>
__device__ __forceinline__ uint32_t gauss_entry_lo(const char* base, uint32_t w) {
  return *reinterpret_cast<const uint32_t*>(base + ((w & 0x3ffu) << SHIFT));
}
template <int SHIFT>
__device__ __forceinline__ uint32_t gauss_entry_hi(const char* base, uint32_t w) {
  return *reinterpret_cast<const uint32_t*>(base + ((w >> (16 - SHIFT)) & (0x3ffu << SHIFT)));
}

// The two normals addressed by the 16-bit halves of `w`, as one bf16x2 register.
template <int SHIFT>
__device__ __forceinline__ uint32_t gauss_pair(const char* base, uint32_t w) {
  const uint32_t e0 = gauss_entry_lo<SHIFT>(base, w), e1 = gauss_entry_hi<SHIFT>(base, w);
  const uint32_t a = __byte_perm(e0, e1, 0x5410), b = __byte_perm(e0, e1, 0x7632);
  const uint32_t m = ((w >> 9) & 0x007E007Eu) | 0x3F813F81u;      // bf16x2 of 1 + (2k + 1) / 128
  uint32_t z;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(z) : "r"(b), "r"(m), "r"(a));
  return z;
}

// The 8 normals of a group as four bf16x2 registers (element 2j in the low half of word j).
template <int SHIFT>
__device__ __forceinline__ void gauss8_packed(const char* base, uint64_t seed, uint32_t tid, uint32_t grp,
                                              uint32_t stream, uint32_t zp[4]) {
  const Philox4 p = z_words(seed, tid, grp, stream);
  zp[0] = gauss_pair<SHIFT>(base, p.x); zp[1] = gauss_pair<SHIFT>(base, p.y);
  zp[2] = gauss_pair<SHIFT>(base, p.z); zp[3] = gauss_pair<SHIFT>(base, p.w);
}

// The same 8 normals widened to fp32.
template <int SHIFT>
__device__ __forceinline__ void gauss8(const char* base, uint64_t seed, uint32_t tid, uint32_t grp,
                                       uint32_t stream, float z[8]) {
  uint32_t zp[4];
  gauss8_packed<SHIFT>(base, seed, tid, grp, stream, zp);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    z[2 * j] = __uint_as_float(zp[j] << 16);
    z[2 * j + 1] = __uint_as_float(zp[j] & 0xffff0000u);
  }
}

// One normal from a 16-bit index and the plain global table (the gamma-search draws).
__device__ __forceinline__ float gauss_scalar(const uint32_t* gtab, uint32_t u16) {
  return __uint_as_float(gauss_pair<2>(reinterpret_cast<const char*>(gtab), u16 & 0xffffu) << 16);
}

// theta + c z for one 16-byte group of bf16 parameters: four fma.rn.bf16x2, each an exact
// product and sum rounded once to bf16.  `c2` holds the coefficient (rounded to bf16) in both halves.
template <int SHIFT>
__device__ __forceinline__ uint4 perturb8_packed(const char* base, uint64_t seed, uint32_t tid,
                                                 uint32_t grp, uint32_t c2, uint4 raw) {
  uint32_t zp[4];
  gauss8_packed<SHIFT>(base, seed, tid, grp, 0u, zp);
  uint32_t v[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; ++j)
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(v[j]) : "r"(c2), "r"(zp[j]), "r"(v[j]));
  return make_uint4(v[0], v[1], v[2], v[3]);
}

// Both signs of the same perturbation from one draw of z: theta + c z and theta - c z (bf16x2, one rounding each).
template <int SHIFT>
__device__ __forceinline__ void perturb8_packed_dual(const char* base, uint64_t seed, uint32_t tid, uint32_t grp,
                                                     uint32_t c2, uint4 raw, uint4& plus, uint4& minus) {
  uint32_t zp[4];
  gauss8_packed<SHIFT>(base, seed, tid, grp, 0u, zp);
  const uint32_t v[4] = {raw.x, raw.y, raw.z, raw.w};
  const uint32_t nc2 = c2 ^ 0x80008000u;          // -c in both halves
  uint32_t a[4], b[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(a[j]) : "r"(c2), "r"(zp[j]), "r"(v[j]));
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(b[j]) : "r"(nc2), "r"(zp[j]), "r"(v[j]));
  }
  plus = make_uint4(a[0], a[1], a[2], a[3]);
  minus = make_uint4(b[0], b[1], b[2], b[3]);
}

// A coefficient rounded to bf16 and replicated into both halves of a bf16x2 register.
__device__ __forceinline__ uint32_t bf16x2_splat(float c) {
  __nv_bfloat162 v = __float2bfloat162_rn(c);
  return *reinterpret_cast<uint32_t*>(&v);
}
#endif

}  // namespace dz
