// LayerNorm and the OPT embedding (token + learned position) for bf16 activations.
//
// layernorm: y = (x - mean) / sqrt(var + eps) * w + b, one CTA per row, the row is held
// in registers between the statistics and the normalisation (one read, one write),
// fp32 statistics with an exact two-pass variance.  Replaces nn.LayerNorm in
// large_models/ht_opt.py:330, :354, :726.
//
// embed: h[m, :] = tok[ids[m], :] + pos[positions[m], :]; positions are the OPT
// convention cumsum(mask) * mask - 1 + 2 and are passed in (large_models/ht_opt.py:114-124,
// :639, :657).
#include "common.cuh"
#include "host_util.h"

namespace dz {

constexpr int LN_MAXV = 4;  // uint4 (8 bf16) per thread held in registers

template <int THREADS>
__global__ void __launch_bounds__(THREADS)
layernorm_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                 const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                 __nv_bfloat16* __restrict__ y, long long ldy, int d, float eps) {
  __shared__ float s_red[THREADS / 32];
  __shared__ float s_bcast;
  const long long row = blockIdx.x;
  const int nvec = d >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  uint4 v[LN_MAXV];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < LN_MAXV; ++i) {
    int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      v[i] = xr[idx];
      sum += bf16_lo(v[i].x) + bf16_hi(v[i].x) + bf16_lo(v[i].y) + bf16_hi(v[i].y) +
             bf16_lo(v[i].z) + bf16_hi(v[i].z) + bf16_lo(v[i].w) + bf16_hi(v[i].w);
    }
  }
  auto block_sum = [&](float val) -> float {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) val += __shfl_xor_sync(0xffffffffu, val, off);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = val;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int k = 0; k < THREADS / 32; ++k) t += s_red[k];
      s_bcast = t;
    }
    __syncthreads();
    float r = s_bcast;
    __syncthreads();
    return r;
  };
  const float mean = block_sum(sum) / d;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < LN_MAXV; ++i) {
    int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      float f[8] = {bf16_lo(v[i].x), bf16_hi(v[i].x), bf16_lo(v[i].y), bf16_hi(v[i].y),
                    bf16_lo(v[i].z), bf16_hi(v[i].z), bf16_lo(v[i].w), bf16_hi(v[i].w)};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float dlt = f[j] - mean;
        sq = fmaf(dlt, dlt, sq);
      }
    }
  }
  const float rstd = rsqrtf(block_sum(sq) / d + eps);
  uint4* yr = reinterpret_cast<uint4*>(y + row * ldy);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const uint4* br = reinterpret_cast<const uint4*>(b);
#pragma unroll
  for (int i = 0; i < LN_MAXV; ++i) {
    int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      uint4 wv = __ldg(wr + idx), bv = __ldg(br + idx);
      uint4 o;
      o.x = pack_bf16x2((bf16_lo(v[i].x) - mean) * rstd * bf16_lo(wv.x) + bf16_lo(bv.x),
                        (bf16_hi(v[i].x) - mean) * rstd * bf16_hi(wv.x) + bf16_hi(bv.x));
      o.y = pack_bf16x2((bf16_lo(v[i].y) - mean) * rstd * bf16_lo(wv.y) + bf16_lo(bv.y),
                        (bf16_hi(v[i].y) - mean) * rstd * bf16_hi(wv.y) + bf16_hi(bv.y));
      o.z = pack_bf16x2((bf16_lo(v[i].z) - mean) * rstd * bf16_lo(wv.z) + bf16_lo(bv.z),
                        (bf16_hi(v[i].z) - mean) * rstd * bf16_hi(wv.z) + bf16_hi(bv.z));
      o.w = pack_bf16x2((bf16_lo(v[i].w) - mean) * rstd * bf16_lo(wv.w) + bf16_lo(bv.w),
                        (bf16_hi(v[i].w) - mean) * rstd * bf16_hi(wv.w) + bf16_hi(bv.w));
      if (DZ_STORE_OK(yr + idx, 16)) yr[idx] = o;
    }
  }
}

__global__ void __launch_bounds__(128)
embed_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
             const __nv_bfloat16* __restrict__ tok, long long ld_tok,
             const __nv_bfloat16* __restrict__ pos, long long ld_pos,
             __nv_bfloat16* __restrict__ out, long long ld_out, int d_tok, int d_pos, int vocab,
             int n_pos) {
  const long long m = blockIdx.x;
  int id = ids[m];
  id = min(max(id, 0), vocab - 1);
  const uint4* tr = reinterpret_cast<const uint4*>(tok + (long long)id * ld_tok);
  uint4* orow = reinterpret_cast<uint4*>(out + m * ld_out);
  if (pos) {
    // token and position rows have the same width: fused add
    int pi = min(max(positions[m], 0), n_pos - 1);
    const uint4* pr = reinterpret_cast<const uint4*>(pos + (long long)pi * ld_pos);
    for (int i = threadIdx.x; i < (d_tok >> 3); i += blockDim.x) {
      uint4 a = __ldg(tr + i), c = __ldg(pr + i), o;
      o.x = pack_bf16x2(bf16_lo(a.x) + bf16_lo(c.x), bf16_hi(a.x) + bf16_hi(c.x));
      o.y = pack_bf16x2(bf16_lo(a.y) + bf16_lo(c.y), bf16_hi(a.y) + bf16_hi(c.y));
      o.z = pack_bf16x2(bf16_lo(a.z) + bf16_lo(c.z), bf16_hi(a.z) + bf16_hi(c.z));
      o.w = pack_bf16x2(bf16_lo(a.w) + bf16_lo(c.w), bf16_hi(a.w) + bf16_hi(c.w));
      if (DZ_STORE_OK(orow + i, 16)) orow[i] = o;
    }
  } else {
    for (int i = threadIdx.x; i < (d_tok >> 3); i += blockDim.x)
      if (DZ_STORE_OK(orow + i, 16)) orow[i] = __ldg(tr + i);
  }
  (void)d_pos;
}

// out[m, :] = a[m, :] + b[idx[m], :]  (bf16): adds position rows after a projection
__global__ void __launch_bounds__(128)
add_rows_kernel(const __nv_bfloat16* __restrict__ a, long long lda, const int* __restrict__ idx,
                const __nv_bfloat16* __restrict__ b, long long ldb, __nv_bfloat16* __restrict__ out,
                long long ldo, int d, int n_b) {
  const long long m = blockIdx.x;
  int bi = min(max(idx[m], 0), n_b - 1);
  const uint4* ar = reinterpret_cast<const uint4*>(a + m * lda);
  const uint4* br = reinterpret_cast<const uint4*>(b + (long long)bi * ldb);
  uint4* orow = reinterpret_cast<uint4*>(out + m * ldo);
  for (int i = threadIdx.x; i < (d >> 3); i += blockDim.x) {
    uint4 x = ar[i], c = __ldg(br + i), o;
    o.x = pack_bf16x2(bf16_lo(x.x) + bf16_lo(c.x), bf16_hi(x.x) + bf16_hi(c.x));
    o.y = pack_bf16x2(bf16_lo(x.y) + bf16_lo(c.y), bf16_hi(x.y) + bf16_hi(c.y));
    o.z = pack_bf16x2(bf16_lo(x.z) + bf16_lo(c.z), bf16_hi(x.z) + bf16_hi(c.z));
    o.w = pack_bf16x2(bf16_lo(x.w) + bf16_lo(c.w), bf16_hi(x.w) + bf16_hi(c.w));
    if (DZ_STORE_OK(orow + i, 16)) orow[i] = o;
  }
}

// out[r, :] = src[rows[r], :]  (bf16 row gather, e.g. the option positions for the LM head)
__global__ void __launch_bounds__(128)
gather_rows_kernel(const __nv_bfloat16* __restrict__ src, long long lds, const int* __restrict__ rows,
                   __nv_bfloat16* __restrict__ out, long long ldo, int d, long long n_src) {
  const long long r = blockIdx.x;
  long long s = rows[r];
  s = s < 0 ? 0 : (s >= n_src ? n_src - 1 : s);
  const uint4* sr = reinterpret_cast<const uint4*>(src + s * lds);
  uint4* orow = reinterpret_cast<uint4*>(out + r * ldo);
  for (int i = threadIdx.x; i < (d >> 3); i += blockDim.x)
    if (DZ_STORE_OK(orow + i, 16)) orow[i] = sr[i];
}

}  // namespace dz

using namespace dz;
DZ_DEBUG_TU(norm)

static bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" int dz_layernorm(const void* x, long long ldx, const void* w, const void* b, void* y,
                            long long ldy, long long rows, int d, float eps, cudaStream_t stream) {
  if (!x || !w || !b || !y || rows <= 0 || d <= 0) return DZ_ERR_ARG;
  if ((d & 7) || (ldx & 7) || (ldy & 7) || !al16(x) || !al16(w) || !al16(b) || !al16(y))
    return DZ_ERR_ALIGN;
  const int nvec = d >> 3;
  auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w;
  auto Bb = (const __nv_bfloat16*)b; auto Y = (__nv_bfloat16*)y;
  if (nvec <= 128 * LN_MAXV)
    layernorm_kernel<128><<<(unsigned)rows, 128, 0, stream>>>(X, ldx, W, Bb, Y, ldy, d, eps);
  else if (nvec <= 256 * LN_MAXV)
    layernorm_kernel<256><<<(unsigned)rows, 256, 0, stream>>>(X, ldx, W, Bb, Y, ldy, d, eps);
  else if (nvec <= 512 * LN_MAXV)
    layernorm_kernel<512><<<(unsigned)rows, 512, 0, stream>>>(X, ldx, W, Bb, Y, ldy, d, eps);
  else
    return DZ_ERR_TOO_LARGE;
  return cuda_rc(cudaGetLastError());
}

extern "C" int dz_embed(const int* ids, const int* positions, const void* tok, long long ld_tok,
                        const void* pos, long long ld_pos, void* out, long long ld_out,
                        long long rows, int d_tok, int vocab, int n_pos, cudaStream_t stream) {
  if (!ids || !tok || !out || rows <= 0 || d_tok <= 0) return DZ_ERR_ARG;
  if (pos && !positions) return DZ_ERR_ARG;
  if ((d_tok & 7) || (ld_tok & 7) || (ld_out & 7) || (pos && (ld_pos & 7)) || !al16(tok) ||
      !al16(out) || (pos && !al16(pos)))
    return DZ_ERR_ALIGN;
  embed_kernel<<<(unsigned)rows, 128, 0, stream>>>(ids, positions, (const __nv_bfloat16*)tok, ld_tok,
                                                   (const __nv_bfloat16*)pos, ld_pos,
                                                   (__nv_bfloat16*)out, ld_out, d_tok, d_tok, vocab,
                                                   n_pos);
  return cuda_rc(cudaGetLastError());
}

extern "C" int dz_add_rows(const void* a, long long lda, const int* idx, const void* b,
                           long long ldb, void* out, long long ldo, long long rows, int d, int n_b,
                           cudaStream_t stream) {
  if (!a || !idx || !b || !out || rows <= 0) return DZ_ERR_ARG;
  if ((d & 7) || (lda & 7) || (ldb & 7) || (ldo & 7) || !al16(a) || !al16(b) || !al16(out))
    return DZ_ERR_ALIGN;
  add_rows_kernel<<<(unsigned)rows, 128, 0, stream>>>((const __nv_bfloat16*)a, lda, idx,
                                                      (const __nv_bfloat16*)b, ldb,
                                                      (__nv_bfloat16*)out, ldo, d, n_b);
  return cuda_rc(cudaGetLastError());
}

extern "C" int dz_gather_rows(const void* src, long long lds, const int* rows_idx, void* out,
                              long long ldo, long long rows, int d, long long n_src,
                              cudaStream_t stream) {
  if (!src || !rows_idx || !out || rows <= 0) return DZ_ERR_ARG;
  if ((d & 7) || (lds & 7) || (ldo & 7) || !al16(src) || !al16(out)) return DZ_ERR_ALIGN;
  gather_rows_kernel<<<(unsigned)rows, 128, 0, stream>>>((const __nv_bfloat16*)src, lds, rows_idx,
                                                         (__nv_bfloat16*)out, ldo, d, n_src);
  return cuda_rc(cudaGetLastError());
}
