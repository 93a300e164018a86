// Memory-bound pieces of the backward pass that the first-order gamma search of DiZO needs
// (large_models/trainer.py:714-741, :805-830 differentiates the loss with respect to the
// per-tensor gamma scalars through autograd): LayerNorm input gradient, the softmax /
// cross-entropy gradient of the LM head rows, a deterministic strided dot product (the
// weight-gradient contraction <dY, X dW^T> of a constrained tensor), row scatter, and the
// element-wise difference theta - theta_0.  The GEMM-shaped parts live in gemm_sm100.cu
// (dz_gemm_bf16_nn) and attn_bwd_sm100.cu.
#include "common.cuh"
#include "host_util.h"

namespace dz {

__device__ __forceinline__ float bk_block_sum(float v, float* red) {
  // every thread of the block calls this; returns the sum to every thread
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  __syncthreads();               // red may still be read from the previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) (+ add),  g = dy * w,  xhat = (x - mean) * rstd.
// One block per row; the row is read from L1/L2 three times.
__global__ void __launch_bounds__(256)
layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, long long lddy, const __nv_bfloat16* __restrict__ x,
                     long long ldx, const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ add,
                     long long ldadd, __nv_bfloat16* __restrict__ dx, long long lddx, int d, float eps) {
  __shared__ float red[8];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * ldx;
  const __nv_bfloat16* gr = dy + row * lddy;
  const int nvec = d >> 3;
  float s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    uint4 v = *reinterpret_cast<const uint4*>(xr + i * 8);
    s += bf16_lo(v.x) + bf16_hi(v.x) + bf16_lo(v.y) + bf16_hi(v.y) + bf16_lo(v.z) + bf16_hi(v.z) +
         bf16_lo(v.w) + bf16_hi(v.w);
  }
  const float mean = bk_block_sum(s, red) / d;
  float s2 = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    uint4 v = *reinterpret_cast<const uint4*>(xr + i * 8);
    float e[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y),
                  bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
#pragma unroll
    for (int j = 0; j < 8; ++j) s2 = fmaf(e[j] - mean, e[j] - mean, s2);
  }
  const float rstd = rsqrtf(bk_block_sum(s2, red) / d + eps);
  float sg = 0.f, sgx = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    uint4 v = *reinterpret_cast<const uint4*>(xr + i * 8);
    uint4 g = *reinterpret_cast<const uint4*>(gr + i * 8);
    uint4 ww = __ldg(reinterpret_cast<const uint4*>(w + i * 8));
    float e[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y),
                  bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
    float gg[8] = {bf16_lo(g.x), bf16_hi(g.x), bf16_lo(g.y), bf16_hi(g.y),
                   bf16_lo(g.z), bf16_hi(g.z), bf16_lo(g.w), bf16_hi(g.w)};
    float we[8] = {bf16_lo(ww.x), bf16_hi(ww.x), bf16_lo(ww.y), bf16_hi(ww.y),
                   bf16_lo(ww.z), bf16_hi(ww.z), bf16_lo(ww.w), bf16_hi(ww.w)};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gw = gg[j] * we[j];
      sg += gw;
      sgx = fmaf(gw, (e[j] - mean) * rstd, sgx);
    }
  }
  const float mg = bk_block_sum(sg, red) / d;
  const float mgx = bk_block_sum(sgx, red) / d;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    uint4 v = *reinterpret_cast<const uint4*>(xr + i * 8);
    uint4 g = *reinterpret_cast<const uint4*>(gr + i * 8);
    uint4 ww = __ldg(reinterpret_cast<const uint4*>(w + i * 8));
    float e[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y),
                  bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
    float gg[8] = {bf16_lo(g.x), bf16_hi(g.x), bf16_lo(g.y), bf16_hi(g.y),
                   bf16_lo(g.z), bf16_hi(g.z), bf16_lo(g.w), bf16_hi(g.w)};
    float we[8] = {bf16_lo(ww.x), bf16_hi(ww.x), bf16_lo(ww.y), bf16_hi(ww.y),
                   bf16_lo(ww.z), bf16_hi(ww.z), bf16_lo(ww.w), bf16_hi(ww.w)};
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = rstd * (gg[j] * we[j] - mg - (e[j] - mean) * rstd * mgx);
    if (add) {
      uint4 a = *reinterpret_cast<const uint4*>(add + row * ldadd + i * 8);
      o[0] += bf16_lo(a.x); o[1] += bf16_hi(a.x); o[2] += bf16_lo(a.y); o[3] += bf16_hi(a.y);
      o[4] += bf16_lo(a.z); o[5] += bf16_hi(a.z); o[6] += bf16_lo(a.w); o[7] += bf16_hi(a.w);
    }
    uint4 r;
    r.x = pack_bf16x2(o[0], o[1]); r.y = pack_bf16x2(o[2], o[3]);
    r.z = pack_bf16x2(o[4], o[5]); r.w = pack_bf16x2(o[6], o[7]);
    uint4* dp = reinterpret_cast<uint4*>(dx + row * lddx + i * 8);
    if (DZ_STORE_OK(dp, 16)) *dp = r;
  }
}

// In place over bf16 logits [R, ldl]: g[r, j] = coef[r] * ((j == target[r]) - exp(logit - lse[r])).
__global__ void __launch_bounds__(256)
softmax_ce_bwd_kernel(__nv_bfloat16* __restrict__ logits, long long ldl, const float* __restrict__ lse,
                      const int* __restrict__ targets, const float* __restrict__ coef, int V) {
  const long long row = blockIdx.y;
  __nv_bfloat16* lr = logits + row * ldl;
  const float l = lse[row], c = coef[row];
  const int t = targets[row];
  const int j0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (j0 >= V) return;
  if (j0 + 8 <= V) {
    uint4 v = *reinterpret_cast<const uint4*>(lr + j0);
    float e[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y),
                  bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = c * ((j0 + j == t ? 1.f : 0.f) - __expf(e[j] - l));
    v.x = pack_bf16x2(e[0], e[1]); v.y = pack_bf16x2(e[2], e[3]);
    v.z = pack_bf16x2(e[4], e[5]); v.w = pack_bf16x2(e[6], e[7]);
    if (DZ_STORE_OK(lr + j0, 16)) *reinterpret_cast<uint4*>(lr + j0) = v;
  } else {
    for (int j = j0; j < V; ++j)
      lr[j] = __float2bfloat16(c * ((j == t ? 1.f : 0.f) - __expf(__bfloat162float(lr[j]) - l)));
  }
}

// partials[block] = sum over the block's share of rows of sum_c a[r, c] * b[r, c]  (fixed order)
constexpr int DOT_BLOCKS = 1024;
__global__ void __launch_bounds__(256)
dot_partial_kernel(const float* __restrict__ a, long long lda, const __nv_bfloat16* __restrict__ b,
                   long long ldb, long long rows, int cols, float* __restrict__ partials) {
  __shared__ float red[8];
  float acc = 0.f;
  const int nvec = cols >> 2;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* ar = a + r * lda;
    const __nv_bfloat16* br = b + r * ldb;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      float4 x = *reinterpret_cast<const float4*>(ar + i * 4);
      uint2 y = *reinterpret_cast<const uint2*>(br + i * 4);
      acc = fmaf(x.x, bf16_lo(y.x), acc);
      acc = fmaf(x.y, bf16_hi(y.x), acc);
      acc = fmaf(x.z, bf16_lo(y.y), acc);
      acc = fmaf(x.w, bf16_hi(y.y), acc);
    }
  }
  const float t = bk_block_sum(acc, red);
  if (threadIdx.x == 0) partials[blockIdx.x] = t;
}

__global__ void __launch_bounds__(256)
dot_final_kernel(const float* __restrict__ partials, int n, float scale, float* __restrict__ out) {
  __shared__ float red[8];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partials[i];
  const float t = bk_block_sum(acc, red);
  if (threadIdx.x == 0) *out = t * scale;
}

__global__ void scatter_rows_kernel(const __nv_bfloat16* __restrict__ src, long long lds,
                                    const int* __restrict__ idx, __nv_bfloat16* __restrict__ dst,
                                    long long ldd, int d, long long n_dst) {
  const long long r = blockIdx.x;
  const long long t = idx[r];
  if (t < 0 || t >= n_dst) return;
  for (int i = threadIdx.x; i < (d >> 3); i += blockDim.x)
    if (DZ_STORE_OK(dst + t * ldd + i * 8, 16))
      *reinterpret_cast<uint4*>(dst + t * ldd + i * 8) = *reinterpret_cast<const uint4*>(src + r * lds + i * 8);
}

__global__ void diff_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                            __nv_bfloat16* __restrict__ out, long long nvec) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    uint4 x = *reinterpret_cast<const uint4*>(a + i * 8);
    uint4 y = *reinterpret_cast<const uint4*>(b + i * 8);
    uint4 r;
    r.x = pack_bf16x2(bf16_lo(x.x) - bf16_lo(y.x), bf16_hi(x.x) - bf16_hi(y.x));
    r.y = pack_bf16x2(bf16_lo(x.y) - bf16_lo(y.y), bf16_hi(x.y) - bf16_hi(y.y));
    r.z = pack_bf16x2(bf16_lo(x.z) - bf16_lo(y.z), bf16_hi(x.z) - bf16_hi(y.z));
    r.w = pack_bf16x2(bf16_lo(x.w) - bf16_lo(y.w), bf16_hi(x.w) - bf16_hi(y.w));
    if (DZ_STORE_OK(out + i * 8, 16)) *reinterpret_cast<uint4*>(out + i * 8) = r;
  }
}

// Prefix rows of the attention backward.  The prefix keys / values are extra key columns that every query sees
// (no mask).  With the forward's log-sum-exp (which covers them) and D = rowsum(dO * O) of the full context,
// their part of the gradient separates from the tiled kernel's:  p = exp2(c q.k_p - lse),  ds = p (dO.v_p - D),
// dQ += scale ds k_p,  dK_p += scale ds q,  dV_p += p dO.  One warp per (batch row, query, head).
__global__ void __launch_bounds__(128)
attn_prefix_bwd_kernel(const __nv_bfloat16* __restrict__ q, long long ldq, const __nv_bfloat16* __restrict__ dout,
                       long long lddo, const __nv_bfloat16* __restrict__ pk, const __nv_bfloat16* __restrict__ pv,
                       long long ldp, int npre, const float* __restrict__ lse, const float* __restrict__ dsum,
                       __nv_bfloat16* __restrict__ dq, long long lddq, float* __restrict__ dpk,
                       float* __restrict__ dpv, long long lddp, int B, int L, int H, int hd, float scale) {
  const long long wid = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)B * L * H) return;
  const int h = (int)(wid % H);
  const long long row = wid / H;                  // b * L + i
  const long long b = row / L, i = row - b * L;
  const float my_lse = lse[(b * H + h) * L + i], my_d = dsum[(b * H + h) * L + i];
  const float c = scale * 1.4426950408889634f;
  float qv[4], gv[4], acc[4];                     // head sizes up to 128: four elements per lane
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int e = lane + 32 * t;
    qv[t] = e < hd ? __bfloat162float(q[row * ldq + h * hd + e]) : 0.f;
    gv[t] = e < hd ? __bfloat162float(dout[row * lddo + h * hd + e]) : 0.f;
    acc[t] = 0.f;
  }
  for (int p = 0; p < npre; ++p) {
    float kv[4], vv[4], s = 0.f, dp = 0.f;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int e = lane + 32 * t;
      kv[t] = e < hd ? __bfloat162float(pk[p * ldp + h * hd + e]) : 0.f;
      vv[t] = e < hd ? __bfloat162float(pv[p * ldp + h * hd + e]) : 0.f;
      s += qv[t] * kv[t];
      dp += gv[t] * vv[t];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, o);
      dp += __shfl_xor_sync(0xffffffffu, dp, o);
    }
    const float prob = exp2f(s * c - my_lse);
    const float ds = prob * (dp - my_d) * scale;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int e = lane + 32 * t;
      acc[t] += ds * kv[t];
      if (dpk && e < hd) {
        atomicAdd(dpk + p * lddp + h * hd + e, ds * qv[t]);
        atomicAdd(dpv + p * lddp + h * hd + e, prob * gv[t]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int e = lane + 32 * t;
    if (e < hd) {
      __nv_bfloat16* o = dq + row * lddq + h * hd + e;
      if (DZ_STORE_OK(o, 2)) *o = __float2bfloat16(__bfloat162float(*o) + acc[t]);
    }
  }
}

static inline bool bk_al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace dz

using namespace dz;
DZ_DEBUG_TU(bwd)

// dx[rows, d] = LayerNorm input gradient for output gradient dy and input x (+ add when given).
extern "C" int dz_layernorm_bwd(const void* dy, long long lddy, const void* x, long long ldx, const void* w,
                                const void* add, long long ldadd, void* dx, long long lddx, long long rows,
                                int d, float eps, cudaStream_t stream) {
  if (!dy || !x || !w || !dx || rows <= 0 || d <= 0) return DZ_ERR_ARG;
  if ((d & 7) || (lddy & 7) || (ldx & 7) || (lddx & 7) || (add && (ldadd & 7)) || !bk_al16(dy) ||
      !bk_al16(x) || !bk_al16(w) || !bk_al16(dx) || (add && !bk_al16(add)))
    return DZ_ERR_ALIGN;
  layernorm_bwd_kernel<<<(unsigned)rows, 256, 0, stream>>>(
      (const __nv_bfloat16*)dy, lddy, (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w,
      (const __nv_bfloat16*)add, ldadd, (__nv_bfloat16*)dx, lddx, d, eps);
  return cuda_rc(cudaGetLastError());
}

// logits [R, ldl] bf16 become coef[r] * (onehot(target[r]) - softmax) in place; lse in natural log.
extern "C" int dz_softmax_ce_bwd(void* logits, long long ldl, const float* lse, const int* targets,
                                 const float* coef, long long rows, int V, cudaStream_t stream) {
  if (!logits || !lse || !targets || !coef || rows <= 0 || V <= 0) return DZ_ERR_ARG;
  if ((ldl & 7) || !bk_al16(logits)) return DZ_ERR_ALIGN;
  if (rows > 65535) return DZ_ERR_TOO_LARGE;
  dim3 grid((V + 2047) / 2048, (unsigned)rows);
  softmax_ce_bwd_kernel<<<grid, 256, 0, stream>>>((__nv_bfloat16*)logits, ldl, lse, targets, coef, V);
  return cuda_rc(cudaGetLastError());
}

// *out = scale * sum_{r, c} a[r, c] * b[r, c]; a fp32 [rows, lda], b bf16 [rows, ldb]; partials is
// fp32 scratch of dz_dot_num_partials() elements.  Fixed reduction order: bitwise reproducible.
extern "C" int dz_dot_num_partials() { return DOT_BLOCKS; }
extern "C" int dz_dot_f32_bf16(const float* a, long long lda, const void* b, long long ldb, long long rows,
                               int cols, float scale, float* partials, float* out, cudaStream_t stream) {
  if (!a || !b || !partials || !out || rows <= 0 || cols <= 0) return DZ_ERR_ARG;
  if ((cols & 3) || (lda & 3) || (ldb & 3) || !bk_al16(a) || (reinterpret_cast<uintptr_t>(b) & 7))
    return DZ_ERR_ALIGN;
  const int blocks = rows < DOT_BLOCKS ? (int)rows : DOT_BLOCKS;
  dot_partial_kernel<<<blocks, 256, 0, stream>>>(a, lda, (const __nv_bfloat16*)b, ldb, rows, cols, partials);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_rc(e);
  dot_final_kernel<<<1, 256, 0, stream>>>(partials, blocks, scale, out);
  return cuda_rc(cudaGetLastError());
}

// dst[idx[r], :] = src[r, :]
extern "C" int dz_scatter_rows(const void* src, long long lds, const int* idx, void* dst, long long ldd,
                               long long rows, int d, long long n_dst, cudaStream_t stream) {
  if (!src || !idx || !dst || rows <= 0) return DZ_ERR_ARG;
  if ((d & 7) || (lds & 7) || (ldd & 7) || !bk_al16(src) || !bk_al16(dst)) return DZ_ERR_ALIGN;
  scatter_rows_kernel<<<(unsigned)rows, 128, 0, stream>>>((const __nv_bfloat16*)src, lds, idx,
                                                          (__nv_bfloat16*)dst, ldd, d, n_dst);
  return cuda_rc(cudaGetLastError());
}

// out = a - b over n bf16 elements (n a multiple of 8)
extern "C" int dz_diff_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t stream) {
  if (!a || !b || !out || n <= 0) return DZ_ERR_ARG;
  if ((n & 7) || !bk_al16(a) || !bk_al16(b) || !bk_al16(out)) return DZ_ERR_ALIGN;
  const long long nvec = n >> 3;
  long long blocks = (nvec + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  diff_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                    (__nv_bfloat16*)out, nvec);
  return cuda_rc(cudaGetLastError());
}

// Adds the prefix rows' part of the attention gradient to dq (bf16 [B*L, lddq], the dQ block that dz_attn_bwd
// wrote) and, when dpk / dpv are given (fp32 [npre, lddp], zeroed by the caller; atomics), accumulates the
// prefix rows' own gradients.  q / dout: bf16 [B*L, ld]; pk / pv: bf16 [npre, ldp]; lse and dsum as dz_attn_bwd.
extern "C" int dz_attn_prefix_bwd(const void* q, long long ldq, const void* dout, long long lddo, const void* pk,
                                  const void* pv, long long ldp, int npre, const float* lse, const float* dsum,
                                  void* dq, long long lddq, float* dpk, float* dpv, long long lddp, int B, int L,
                                  int H, int hd, float scale, cudaStream_t stream) {
  if (!q || !dout || !pk || !pv || !lse || !dsum || !dq || B <= 0 || L <= 0 || H <= 0 || npre <= 0)
    return DZ_ERR_ARG;
  if (hd <= 0 || hd > 128 || (dpk == nullptr) != (dpv == nullptr)) return DZ_ERR_ARG;
  const long long warps = (long long)B * L * H;
  if ((warps + 3) / 4 > 0x7fffffffLL) return DZ_ERR_TOO_LARGE;
  attn_prefix_bwd_kernel<<<(unsigned)((warps + 3) / 4), 128, 0, stream>>>(
      (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)dout, lddo, (const __nv_bfloat16*)pk,
      (const __nv_bfloat16*)pv, ldp, npre, lse, dsum, (__nv_bfloat16*)dq, lddq, dpk, dpv, lddp, B, L, H, hd, scale);
  return cuda_rc(cudaGetLastError());
}
