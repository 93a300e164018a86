// Generation-time kernels: single-token attention over a KV cache and token sampling.
//
// decode_attn: one new query per sequence against the cached keys / values (plus optional
// prefix rows); one CTA per (sequence, head); scores in shared memory, fp32 softmax.
// Bandwidth-bound (every cached K and V element is read once).
//
// sample_topk_topp: temperature -> top-k -> nucleus (top-p) filtering and one draw per row,
// without sorting the vocabulary: the k-th largest logit and the nucleus threshold are found
// by bisection on the value (each step is one block-wide count / mass reduction), the draw
// walks the kept probability mass with a uniform from Philox(seed, row).  Semantics follow
// Hugging Face's logits warpers (temperature, TopK, TopP in that order), which is what the
// reference's model.generate applies (large_models/run.py:280-287).
#include "common.cuh"
#include "host_util.h"
#include "philox.cuh"

namespace dz {

constexpr int DA_THREADS = 256;
constexpr int DA_WARPS = DA_THREADS / 32;
constexpr int DA_UNROLL = 4;      // independent cache rows in flight per thread

__global__ void __launch_bounds__(DA_THREADS)
decode_attn_kernel(const __nv_bfloat16* __restrict__ q, long long ldq,
                   const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                   long long ld_seq, long long ld_row,  // cache strides: per sequence, per position
                   const __nv_bfloat16* __restrict__ pk, const __nv_bfloat16* __restrict__ pv,
                   long long ldp, int n_prefix, const int* __restrict__ pad_left, int kv_len, int hd,
                   float scale, __nv_bfloat16* __restrict__ out, long long ldo) {
  extern __shared__ float s_score[];          // [n_prefix + kv_len]
  __shared__ float s_red[DA_WARPS];
  __shared__ float s_q[128];
  __shared__ float s_part[DA_WARPS][128];     // per-warp partial outputs
  const int b = blockIdx.y, h = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pad = pad_left ? pad_left[b] : 0;
  const int total = n_prefix + kv_len;
  if (tid < hd) s_q[tid] = __bfloat162float(q[(long long)b * ldq + h * hd + tid]) * scale;
  __syncthreads();
  const __nv_bfloat16* kbase = kc + (long long)b * ld_seq + h * hd;
  const __nv_bfloat16* vbase = vc + (long long)b * ld_seq + h * hd;
  // ---- scores: a half-warp per key (16 lanes x 8 elements cover hd <= 128), DA_UNROLL keys of
  // each half-warp in flight.  The trip count is the same for every lane of a warp (the shuffles
  // need all 32 lanes).
  const int sub = lane >> 4, l16 = lane & 15;
  const bool col_ok = l16 * 8 < hd;
  float lmax = -INFINITY;
  for (int jb = warp * 2; jb < total; jb += DA_WARPS * 2 * DA_UNROLL) {
    uint4 kv[DA_UNROLL];
#pragma unroll
    for (int u = 0; u < DA_UNROLL; ++u) {
      const int j = jb + u * DA_WARPS * 2 + sub;
      kv[u] = make_uint4(0u, 0u, 0u, 0u);
      if (j < total && col_ok) {
        const __nv_bfloat16* krow = j < n_prefix ? pk + (long long)j * ldp + h * hd
                                                 : kbase + (long long)(j - n_prefix) * ld_row;
        kv[u] = *reinterpret_cast<const uint4*>(krow + l16 * 8);
      }
    }
    const float* qq = s_q + l16 * 8;
#pragma unroll
    for (int u = 0; u < DA_UNROLL; ++u) {
      const int j = jb + u * DA_WARPS * 2 + sub;
      float acc = 0.f;
      if (col_ok)
        acc = qq[0] * bf16_lo(kv[u].x) + qq[1] * bf16_hi(kv[u].x) + qq[2] * bf16_lo(kv[u].y) +
              qq[3] * bf16_hi(kv[u].y) + qq[4] * bf16_lo(kv[u].z) + qq[5] * bf16_hi(kv[u].z) +
              qq[6] * bf16_lo(kv[u].w) + qq[7] * bf16_hi(kv[u].w);
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (j < total) {
        const bool vis = j < n_prefix || (j - n_prefix) >= pad;
        if (!vis) acc = -INFINITY;
        if (l16 == 0) s_score[j] = acc;
        lmax = fmaxf(lmax, acc);
      }
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, off));
  if (lane == 0) s_red[warp] = lmax;
  __syncthreads();
  float m = s_red[0];
  for (int w = 1; w < DA_WARPS; ++w) m = fmaxf(m, s_red[w]);
  __syncthreads();
  float lsum = 0.f;
  for (int j = tid; j < total; j += DA_THREADS) {
    float e = __expf(s_score[j] - m);
    s_score[j] = e;
    lsum += e;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, off);
  if (lane == 0) s_red[warp] = lsum;
  __syncthreads();
  float denom = 0.f;
  for (int w = 0; w < DA_WARPS; ++w) denom += s_red[w];
  // ---- output: warp w takes keys w, w + 8, ...; lane l the columns [4l, 4l + 4); DA_UNROLL rows
  // in flight; the warps' partial sums meet in shared memory.
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const bool vcol_ok = lane * 4 < hd;
  for (int jb = warp; jb < total; jb += DA_WARPS * DA_UNROLL) {
    uint2 vv[DA_UNROLL];
    float pj[DA_UNROLL];
#pragma unroll
    for (int u = 0; u < DA_UNROLL; ++u) {
      const int j = jb + u * DA_WARPS;
      vv[u] = make_uint2(0u, 0u);
      pj[u] = 0.f;
      if (j < total) {
        pj[u] = s_score[j];
        if (vcol_ok) {
          const __nv_bfloat16* vrow = j < n_prefix ? pv + (long long)j * ldp + h * hd
                                                   : vbase + (long long)(j - n_prefix) * ld_row;
          vv[u] = *reinterpret_cast<const uint2*>(vrow + lane * 4);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < DA_UNROLL; ++u) {
      acc[0] = fmaf(pj[u], bf16_lo(vv[u].x), acc[0]);
      acc[1] = fmaf(pj[u], bf16_hi(vv[u].x), acc[1]);
      acc[2] = fmaf(pj[u], bf16_lo(vv[u].y), acc[2]);
      acc[3] = fmaf(pj[u], bf16_hi(vv[u].y), acc[3]);
    }
  }
  if (vcol_ok) {
#pragma unroll
    for (int c = 0; c < 4; ++c) s_part[warp][lane * 4 + c] = acc[c];
  }
  __syncthreads();
  if (tid < hd) {
    float o = 0.f;
    for (int w = 0; w < DA_WARPS; ++w) o += s_part[w][tid];
    out[(long long)b * ldo + h * hd + tid] = __float2bfloat16(o / denom);
  }
}

constexpr int SP_THREADS = 512;

__device__ __forceinline__ float block_sum(float v, float* s_red) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < SP_THREADS / 32; ++w) t += s_red[w];
  __syncthreads();
  return t;
}
__device__ __forceinline__ float block_max(float v, float* s_red) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = -INFINITY;
  for (int w = 0; w < SP_THREADS / 32; ++w) t = fmaxf(t, s_red[w]);
  __syncthreads();
  return t;
}

// One CTA per row.  do_sample == 0: argmax.
__global__ void __launch_bounds__(SP_THREADS)
sample_topk_topp_kernel(const float* __restrict__ logits, long long ld, int V, float temperature,
                        int top_k, float top_p, int do_sample, unsigned long long seed,
                        unsigned long long offset, int* __restrict__ out) {
  __shared__ float s_red[SP_THREADS / 32];
  __shared__ int s_idx[SP_THREADS / 32];
  __shared__ float s_chunk[SP_THREADS];
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* lg = logits + (long long)row * ld;
  const float inv_t = (do_sample && temperature > 0.f) ? 1.0f / temperature : 1.0f;
  // ---- maximum (and argmax with the lowest index on ties)
  float best = -INFINITY;
  int best_i = V;
  for (int i = tid; i < V; i += SP_THREADS) {
    float x = lg[i] * inv_t;
    if (x > best) { best = x; best_i = i; }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    float ob = __shfl_xor_sync(0xffffffffu, best, off);
    int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
    if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
  }
  if ((tid & 31) == 0) { s_red[tid >> 5] = best; s_idx[tid >> 5] = best_i; }
  __syncthreads();
  float m = s_red[0];
  int mi = s_idx[0];
  for (int w = 1; w < SP_THREADS / 32; ++w)
    if (s_red[w] > m || (s_red[w] == m && s_idx[w] < mi)) { m = s_red[w]; mi = s_idx[w]; }
  __syncthreads();
  if (!do_sample) {
    if (tid == 0) out[row] = mi;
    return;
  }
  // ---- top-k: smallest logit that is still kept = k-th largest, by bisection on the value
  float lo_keep = -INFINITY;
  if (top_k > 0 && top_k < V) {
    float lo = m - 60.f, hi = m;                     // logits more than 60 below the max carry no mass
    for (int it = 0; it < 32; ++it) {
      float mid = 0.5f * (lo + hi);
      float c = 0.f;
      for (int i = tid; i < V; i += SP_THREADS) c += (lg[i] * inv_t >= mid) ? 1.f : 0.f;
      c = block_sum(c, s_red);
      if (c >= (float)top_k) lo = mid; else hi = mid;  // keep at least k tokens at threshold lo
    }
    lo_keep = lo;
  }
  // ---- normaliser of the top-k set
  float z = 0.f;
  for (int i = tid; i < V; i += SP_THREADS) {
    float x = lg[i] * inv_t;
    if (x >= lo_keep) z += __expf(x - m);
  }
  z = block_sum(z, s_red);
  // ---- nucleus: largest threshold whose kept mass still reaches top_p
  float p_keep = 0.f;                                // keep probabilities >= p_keep
  if (top_p > 0.f && top_p < 1.f) {
    float lo = 0.f, hi = 1.0f;
    for (int it = 0; it < 32; ++it) {
      float mid = 0.5f * (lo + hi);
      float mass = 0.f;
      for (int i = tid; i < V; i += SP_THREADS) {
        float x = lg[i] * inv_t;
        if (x >= lo_keep) {
          float pr = __expf(x - m) / z;
          if (pr >= mid) mass += pr;
        }
      }
      mass = block_sum(mass, s_red);
      if (mass >= top_p) lo = mid; else hi = mid;
    }
    p_keep = lo;
  }
  // ---- kept mass, then walk it with one uniform
  float kept = 0.f;
  for (int i = tid; i < V; i += SP_THREADS) {
    float x = lg[i] * inv_t;
    if (x >= lo_keep) {
      float pr = __expf(x - m) / z;
      if (pr >= p_keep) kept += pr;
    }
  }
  kept = block_sum(kept, s_red);
  Philox4 r = philox4x32<10>((uint32_t)row, (uint32_t)offset, (uint32_t)(offset >> 32), 3u,
                             (uint32_t)seed, (uint32_t)(seed >> 32));
  const float u = ((r.x >> 8) + 0.5f) * (1.0f / 16777216.0f) * kept;
  float run = 0.f;
  int chosen = mi;
  bool found = false;
  for (int base = 0; base < V && !found; base += SP_THREADS) {
    int i = base + tid;
    float pr = 0.f;
    if (i < V) {
      float x = lg[i] * inv_t;
      if (x >= lo_keep) {
        float q = __expf(x - m) / z;
        if (q >= p_keep) pr = q;
      }
    }
    s_chunk[tid] = pr;
    __syncthreads();
    if (tid == 0) {
      for (int t = 0; t < SP_THREADS; ++t) {
        run += s_chunk[t];
        if (s_chunk[t] > 0.f && run >= u) { s_idx[0] = base + t; s_red[0] = 1.f; break; }
        if (t == SP_THREADS - 1) s_red[0] = 0.f;
      }
      s_red[1] = run;
    }
    __syncthreads();
    found = s_red[0] > 0.5f;
    run = s_red[1];
    if (found) chosen = s_idx[0];
    __syncthreads();
  }
  if (tid == 0) out[row] = chosen;
}

}  // namespace dz

using namespace dz;

extern "C" int dz_decode_attn(const void* q, long long ldq, const void* kc, const void* vc,
                              long long ld_seq, long long ld_row, const void* pk, const void* pv,
                              long long ldp, int n_prefix, const int* pad_left, int kv_len, int B,
                              int H, int hd, float scale, void* out, long long ldo,
                              cudaStream_t stream) {
  if (!q || !kc || !vc || !out || B <= 0 || H <= 0 || kv_len <= 0) return DZ_ERR_ARG;
  if (hd > 128 || (hd & 7) || (ld_row & 7) || (ld_seq & 7) || (n_prefix > 0 && (!pk || !pv || (ldp & 7))))
    return DZ_ERR_ARG;
  size_t smem = sizeof(float) * (size_t)(n_prefix + kv_len);
  if (smem > 160 * 1024) return DZ_ERR_TOO_LARGE;
  static PerDeviceFlag configured;
  if (int rc_cfg = ensure_dyn_smem(configured, decode_attn_kernel, 160 * 1024)) return rc_cfg;
  dim3 grid(H, B);
  decode_attn_kernel<<<grid, DA_THREADS, smem, stream>>>(
      (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, ld_seq, ld_row,
      (const __nv_bfloat16*)pk, (const __nv_bfloat16*)pv, ldp, n_prefix, pad_left, kv_len, hd, scale,
      (__nv_bfloat16*)out, ldo);
  return cuda_rc(cudaGetLastError());
}

extern "C" int dz_sample_topk_topp(const float* logits, long long ld, int rows, int V, float temperature,
                                   int top_k, float top_p, int do_sample, unsigned long long seed,
                                   unsigned long long offset, int* out, cudaStream_t stream) {
  if (!logits || !out || rows <= 0 || V <= 0) return DZ_ERR_ARG;
  sample_topk_topp_kernel<<<rows, SP_THREADS, 0, stream>>>(logits, ld, V, temperature, top_k, top_p,
                                                           do_sample, seed, offset, out);
  return cuda_rc(cudaGetLastError());
}
