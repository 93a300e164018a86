// Counter-based Gaussian stream shared by every kernel that needs the perturbation z.
//
// z for element e of tensor t under seed s is a pure function of (s, t, e):
//   words  = Philox4x32-10(counter = (e >> 3, t, stream, 0), key = (s_lo, s_hi))
//   word j = words[(e & 7) >> 1]; u1 = word & 0xffff, u2 = word >> 16
//   r = sqrt(-2 ln((u1 + 0.5) / 65536)),  phi = 2 pi (u2 + 0.5) / 65536 - pi
//   z = r cos(phi) if e is even, r sin(phi) if e is odd
// so one Philox call yields the 8 normals of one 16-byte group of bf16 parameters, z is
// never stored, and any sharding of a tensor (data-, tensor- or fully-sharded-parallel)
// sees the same values.  The reference instead re-seeds torch's generator and
// materialises z per tensor (large_models/trainer.py:1438-1444, :1603-1608).
#pragma once
#include <stdint.h>

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
#ifdef __CUDA_ARCH__
    uint32_t hi0 = __umulhi(PHILOX_M0, c0);
    uint32_t hi1 = __umulhi(PHILOX_M1, c2);
#else
    uint32_t hi0 = (uint32_t)(((uint64_t)PHILOX_M0 * c0) >> 32);
    uint32_t hi1 = (uint32_t)(((uint64_t)PHILOX_M1 * c2) >> 32);
#endif
    uint32_t lo0 = PHILOX_M0 * c0;
    uint32_t lo1 = PHILOX_M1 * c2;
    uint32_t n0 = hi1 ^ c1 ^ k0;
    uint32_t n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += PHILOX_W0;
    k1 += PHILOX_W1;
  }
  return Philox4{c0, c1, c2, c3};
}

#ifdef __CUDACC__
// Two normals from one 32-bit word (Box-Muller on two 16-bit uniforms).
__device__ __forceinline__ void gauss_pair(uint32_t word, float& z0, float& z1) {
  const float u1 = (static_cast<float>(word & 0xffffu) + 0.5f) * (1.0f / 65536.0f);
  const float u2 = static_cast<float>(word >> 16) + 0.5f;
  // -2 ln(u1) = -2 ln2 * log2(u1)
  const float r = sqrtf(-1.3862943611198906f * __log2f(u1));
  const float phi = u2 * (6.283185307179586f / 65536.0f) - 3.141592653589793f;
  float s, c;
  __sincosf(phi, &s, &c);
  z0 = r * c;
  z1 = r * s;
}

// The 8 normals of group `grp` (= element index >> 3) of tensor `tid`.
__device__ __forceinline__ void gauss8(uint64_t seed, uint32_t tid, uint32_t grp, uint32_t stream,
                                       float z[8]) {
  Philox4 p = philox4x32<10>(grp, tid, stream, 0u, static_cast<uint32_t>(seed),
                             static_cast<uint32_t>(seed >> 32));
  gauss_pair(p.x, z[0], z[1]);
  gauss_pair(p.y, z[2], z[3]);
  gauss_pair(p.z, z[4], z[5]);
  gauss_pair(p.w, z[6], z[7]);
}
#endif

}  // namespace dz
