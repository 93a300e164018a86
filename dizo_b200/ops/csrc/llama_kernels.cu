// Memory-bound pieces of the LLaMA-family decoder block (RMSNorm, rotary position embedding with the
// key / value heads of grouped-query attention expanded, SwiGLU gate) for bf16 activations.  The
// reference reaches these models through Hugging Face modules (large_models/run.py:167-181 loads any
// causal LM; :242-265 and large_models/prefix.py:112-125 name the llama head and attention modules).
//
// rmsnorm : y = x * rsqrt(mean(x^2) + eps) * w, one CTA per row, the row held in registers (one read,
//           one write), fp32 statistics.
// rope_qkv: the fused projection output [q (H*hd) | k (Hkv*hd) | v (Hkv*hd)] of a row becomes the
//           [q | k | v] layout (3*H*hd) the attention kernels read: q and k rotated by the row's position
//           (pairs (j, j + hd/2), angle = position * theta^(-2j/hd), cos / sin from a host-built fp32
//           table so that large angles keep full precision), k and v heads repeated H / Hkv times.
// silu_mul: out[m, f] = silu(gu[m, f]) * gu[m, F + f] for the fused gate | up projection output.
#include "common.cuh"
#include "host_util.h"

namespace dz {

constexpr int RMS_MAXV = 4;  // uint4 (8 bf16) per thread held in registers

template <int THREADS>
__global__ void __launch_bounds__(THREADS)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w,
               __nv_bfloat16* __restrict__ y, long long ldy, int d, float eps) {
  __shared__ float s_red[THREADS / 32];
  const long long row = blockIdx.x;
  const int nvec = d >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  uint4 v[RMS_MAXV];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < RMS_MAXV; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      v[i] = xr[idx];
      const float f[8] = {bf16_lo(v[i].x), bf16_hi(v[i].x), bf16_lo(v[i].y), bf16_hi(v[i].y),
                          bf16_lo(v[i].z), bf16_hi(v[i].z), bf16_lo(v[i].w), bf16_hi(v[i].w)};
#pragma unroll
      for (int j = 0; j < 8; ++j) sq = fmaf(f[j], f[j], sq);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = sq;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int k = 0; k < THREADS / 32; ++k) tot += s_red[k];
  const float rstd = rsqrtf(tot / d + eps);
  uint4* yr = reinterpret_cast<uint4*>(y + row * ldy);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int i = 0; i < RMS_MAXV; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      const uint4 wv = __ldg(wr + idx);
      uint4 o;
      o.x = pack_bf16x2(bf16_lo(v[i].x) * rstd * bf16_lo(wv.x), bf16_hi(v[i].x) * rstd * bf16_hi(wv.x));
      o.y = pack_bf16x2(bf16_lo(v[i].y) * rstd * bf16_lo(wv.y), bf16_hi(v[i].y) * rstd * bf16_hi(wv.y));
      o.z = pack_bf16x2(bf16_lo(v[i].z) * rstd * bf16_lo(wv.z), bf16_hi(v[i].z) * rstd * bf16_hi(wv.z));
      o.w = pack_bf16x2(bf16_lo(v[i].w) * rstd * bf16_lo(wv.w), bf16_hi(v[i].w) * rstd * bf16_hi(wv.w));
      if (DZ_STORE_OK(yr + idx, 16)) yr[idx] = o;
    }
  }
}

// One work item = two adjacent rotary pairs of one head: elements (j0, j0 + 1) and (j0 + hd/2, j0 + hd/2 + 1).
__global__ void __launch_bounds__(256)
rope_qkv_kernel(const __nv_bfloat16* __restrict__ in, long long ld_in, __nv_bfloat16* __restrict__ out,
                long long ld_out, const float2* __restrict__ cs, int L, int pos0, int n_pos, int H, int Hkv,
                int hd) {
  const long long row = blockIdx.x;
  const int half = hd >> 1;
  const int per_head = hd >> 2;
  const int items = 3 * H * per_head;
  int pos = pos0 + (int)(row % L);
  pos = pos < n_pos ? pos : n_pos - 1;                  // the host sizes the table; never read past it
  const float2* csr = cs + (long long)pos * half;
  const __nv_bfloat16* ir = in + row * ld_in;
  __nv_bfloat16* orow = out + row * ld_out;
  const int rep = H / Hkv;
  for (int it = threadIdx.x; it < items; it += blockDim.x) {
    const int sec = it / (H * per_head);                // 0 q, 1 k, 2 v
    const int r = it - sec * H * per_head;
    const int h = r / per_head;
    const int j0 = (r - h * per_head) * 2;
    const int src_h = sec == 0 ? h : h / rep;
    const int src_base = (sec == 0 ? 0 : (sec == 1 ? H * hd : (H + Hkv) * hd)) + src_h * hd;
    const uint32_t lo = *reinterpret_cast<const uint32_t*>(ir + src_base + j0);
    const uint32_t hi = *reinterpret_cast<const uint32_t*>(ir + src_base + half + j0);
    uint32_t o_lo = lo, o_hi = hi;
    if (sec < 2) {
      const float2 c0 = __ldg(csr + j0), c1 = __ldg(csr + j0 + 1);      // (cos, sin)
      const float a0 = bf16_lo(lo), a1 = bf16_hi(lo), b0 = bf16_lo(hi), b1 = bf16_hi(hi);
      o_lo = pack_bf16x2(a0 * c0.x - b0 * c0.y, a1 * c1.x - b1 * c1.y);
      o_hi = pack_bf16x2(b0 * c0.x + a0 * c0.y, b1 * c1.x + a1 * c1.y);
    }
    __nv_bfloat16* dst = orow + (sec * H + h) * hd + j0;
    if (DZ_STORE_OK(dst, 4)) *reinterpret_cast<uint32_t*>(dst) = o_lo;
    if (DZ_STORE_OK(dst + half, 4)) *reinterpret_cast<uint32_t*>(dst + half) = o_hi;
  }
}

__global__ void __launch_bounds__(256)
silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, long long ld, __nv_bfloat16* __restrict__ out,
                long long ldo, long long rows, int F) {
  const int nvec = F >> 3;
  const long long total = rows * nvec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / nvec;
    const int c = (int)(i - r * nvec) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + r * ld + c);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + r * ld + F + c);
    auto f = [](float a, float b) { return a / (1.f + __expf(-a)) * b; };
    uint4 o;
    o.x = pack_bf16x2(f(bf16_lo(g.x), bf16_lo(u.x)), f(bf16_hi(g.x), bf16_hi(u.x)));
    o.y = pack_bf16x2(f(bf16_lo(g.y), bf16_lo(u.y)), f(bf16_hi(g.y), bf16_hi(u.y)));
    o.z = pack_bf16x2(f(bf16_lo(g.z), bf16_lo(u.z)), f(bf16_hi(g.z), bf16_hi(u.z)));
    o.w = pack_bf16x2(f(bf16_lo(g.w), bf16_lo(u.w)), f(bf16_hi(g.w), bf16_hi(u.w)));
    if (DZ_STORE_OK(out + r * ldo + c, 16)) *reinterpret_cast<uint4*>(out + r * ldo + c) = o;
  }
}

static inline bool lk_al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace dz

using namespace dz;
DZ_DEBUG_TU(llama)

extern "C" int dz_rmsnorm(const void* x, long long ldx, const void* w, void* y, long long ldy, long long rows,
                          int d, float eps, cudaStream_t stream) {
  if (!x || !w || !y || rows <= 0 || d <= 0) return DZ_ERR_ARG;
  if ((d & 7) || (ldx & 7) || (ldy & 7) || !lk_al16(x) || !lk_al16(w) || !lk_al16(y)) return DZ_ERR_ALIGN;
  const int nvec = d >> 3;
  auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w; auto Y = (__nv_bfloat16*)y;
  if (nvec <= 128 * RMS_MAXV)
    rmsnorm_kernel<128><<<(unsigned)rows, 128, 0, stream>>>(X, ldx, W, Y, ldy, d, eps);
  else if (nvec <= 256 * RMS_MAXV)
    rmsnorm_kernel<256><<<(unsigned)rows, 256, 0, stream>>>(X, ldx, W, Y, ldy, d, eps);
  else if (nvec <= 512 * RMS_MAXV)
    rmsnorm_kernel<512><<<(unsigned)rows, 512, 0, stream>>>(X, ldx, W, Y, ldy, d, eps);
  else
    return DZ_ERR_TOO_LARGE;
  return cuda_rc(cudaGetLastError());
}

// in: bf16 [rows, ld_in] holding q (H*hd) | k (Hkv*hd) | v (Hkv*hd); out: bf16 [rows, ld_out] holding
// q | k | v of H heads each; cs: fp32 (cos, sin) [n_pos, hd/2]; the position of row m is pos0 + m % L.
extern "C" int dz_rope_qkv(const void* in, long long ld_in, void* out, long long ld_out, const void* cs,
                           long long rows, int L, int pos0, int n_pos, int H, int Hkv, int hd,
                           cudaStream_t stream) {
  if (!in || !out || !cs || rows <= 0 || L <= 0 || H <= 0 || Hkv <= 0 || hd <= 0 || n_pos <= 0 || pos0 < 0)
    return DZ_ERR_ARG;
  if ((hd & 3) || (H % Hkv) || (ld_in & 1) || (ld_out & 1)) return DZ_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(in) & 3) || (reinterpret_cast<uintptr_t>(out) & 3) ||
      (reinterpret_cast<uintptr_t>(cs) & 7))
    return DZ_ERR_ALIGN;
  if (rows > 0x7fffffffLL) return DZ_ERR_TOO_LARGE;
  rope_qkv_kernel<<<(unsigned)rows, 256, 0, stream>>>((const __nv_bfloat16*)in, ld_in, (__nv_bfloat16*)out,
                                                       ld_out, (const float2*)cs, L, pos0, n_pos, H, Hkv, hd);
  return cuda_rc(cudaGetLastError());
}

// gu: bf16 [rows, ld] holding gate (F) | up (F); out: bf16 [rows, ldo] = silu(gate) * up.
extern "C" int dz_silu_mul(const void* gu, long long ld, void* out, long long ldo, long long rows, int F,
                           cudaStream_t stream) {
  if (!gu || !out || rows <= 0 || F <= 0) return DZ_ERR_ARG;
  if ((F & 7) || (ld & 7) || (ldo & 7) || !lk_al16(gu) || !lk_al16(out)) return DZ_ERR_ALIGN;
  long long blocks = (rows * (F >> 3) + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  silu_mul_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)gu, ld, (__nv_bfloat16*)out, ldo,
                                                         rows, F);
  return cuda_rc(cudaGetLastError());
}
