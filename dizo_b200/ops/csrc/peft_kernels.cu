// LoRA merge for forward-only training:  out[n, k] = W[n, k] + s * sum_r B[n, r] * A[r, k].
//
// Zeroth-order training never back-propagates, so the low-rank update can be folded into
// the projection weight before the (single, full-speed) QKV GEMM instead of running the two
// skinny GEMMs x A^T B^T of the reference (large_models/lora.py:89-98).  The merge is one
// bandwidth-bound pass over the d x d weight (read W, write the staged W_eff), r <= 16.
#include "common.cuh"
#include "host_util.h"

namespace dz {

constexpr int LORA_MAX_R = 16;

template <int R>
__global__ void __launch_bounds__(256)
lora_merge_kernel(const __nv_bfloat16* __restrict__ W, long long ldw,
                  const __nv_bfloat16* __restrict__ A, long long lda,   // [R, K]
                  const __nv_bfloat16* __restrict__ B, long long ldb,   // [N, R]
                  __nv_bfloat16* __restrict__ out, long long ldo, int N, int K, float s) {
  // grid: (ceil(K / 2048), N); each thread owns 8 consecutive k of one row n
  const int n = blockIdx.y;
  const int k0 = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (k0 >= K) return;
  float b[R];
#pragma unroll
  for (int r = 0; r < R; ++r) b[r] = s * __bfloat162float(B[(long long)n * ldb + r]);
  uint4 w = *reinterpret_cast<const uint4*>(W + (long long)n * ldw + k0);
  float v[8] = {bf16_lo(w.x), bf16_hi(w.x), bf16_lo(w.y), bf16_hi(w.y),
                bf16_lo(w.z), bf16_hi(w.z), bf16_lo(w.w), bf16_hi(w.w)};
#pragma unroll
  for (int r = 0; r < R; ++r) {
    uint4 a = __ldg(reinterpret_cast<const uint4*>(A + (long long)r * lda + k0));
    v[0] = fmaf(b[r], bf16_lo(a.x), v[0]); v[1] = fmaf(b[r], bf16_hi(a.x), v[1]);
    v[2] = fmaf(b[r], bf16_lo(a.y), v[2]); v[3] = fmaf(b[r], bf16_hi(a.y), v[3]);
    v[4] = fmaf(b[r], bf16_lo(a.z), v[4]); v[5] = fmaf(b[r], bf16_hi(a.z), v[5]);
    v[6] = fmaf(b[r], bf16_lo(a.w), v[6]); v[7] = fmaf(b[r], bf16_hi(a.w), v[7]);
  }
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
  if (DZ_STORE_OK(out + (long long)n * ldo + k0, 16)) *reinterpret_cast<uint4*>(out + (long long)n * ldo + k0) = o;
}

}  // namespace dz

using namespace dz;
DZ_DEBUG_TU(peft)

extern "C" int dz_lora_merge(const void* W, long long ldw, const void* A, long long lda,
                             const void* B, long long ldb, void* out, long long ldo, int N, int K,
                             int r, float scaling, cudaStream_t stream) {
  if (!W || !A || !B || !out || N <= 0 || K <= 0 || r <= 0) return DZ_ERR_ARG;
  if (r > LORA_MAX_R) return DZ_ERR_TOO_LARGE;
  if ((K & 7) || (ldw & 7) || (lda & 7) || (ldo & 7) || (reinterpret_cast<uintptr_t>(W) & 15) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return DZ_ERR_ALIGN;
  dim3 grid((K + 2047) / 2048, N);
  auto w = (const __nv_bfloat16*)W; auto a = (const __nv_bfloat16*)A;
  auto b = (const __nv_bfloat16*)B; auto o = (__nv_bfloat16*)out;
  switch (r) {
#define DZ_R(RR) case RR: lora_merge_kernel<RR><<<grid, 256, 0, stream>>>(w, ldw, a, lda, b, ldb, o, ldo, N, K, scaling); break;
    DZ_R(1) DZ_R(2) DZ_R(3) DZ_R(4) DZ_R(5) DZ_R(6) DZ_R(7) DZ_R(8)
    DZ_R(9) DZ_R(10) DZ_R(11) DZ_R(12) DZ_R(13) DZ_R(14) DZ_R(15) DZ_R(16)
#undef DZ_R
  }
  return cuda_rc(cudaGetLastError());
}
