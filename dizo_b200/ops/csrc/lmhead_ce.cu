// Loss tail of the forward pass: everything after the final LayerNorm.
//
// The reference computes logits for every position ([B, L, V] in fp16), shifts, runs a
// full-vocabulary log_softmax, gathers the gold tokens, averages the last `option_len`
// of them per candidate and takes a cross entropy over the candidates
// (large_models/ht_opt.py:956, large_models/trainer.py:1469-1510).  Here:
//   * only the rows that predict option tokens are multiplied with the embedding table
//     (dz_gemm_bf16_tn_lse: the GEMM epilogue keeps an online log-sum-exp per row and
//     picks up the gold logit, no [rows, V] tensor is written);
//   * dz_lse_combine merges the per-column-tile partials into log p(gold) per row;
//   * dz_option_ce turns the rows into one fp32 loss on the device (candidate mean,
//     cross entropy over candidates, mean over examples; or plain token cross entropy);
//   * dz_verbalizer_ce is the shortcut for single-token candidates that share their
//     prompt: CE over the last-position logits of the candidate ids only.
#include "common.cuh"
#include "host_util.h"

namespace dz {

__global__ void lse_combine_kernel(const float* __restrict__ part_max,
                                   const float* __restrict__ part_sum,
                                   const float* __restrict__ tgt_logit, int num_tiles, int rows,
                                   float* __restrict__ logprob, float* __restrict__ lse_out) {
  int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const float* pm = part_max + (long long)r * num_tiles;
  const float* ps = part_sum + (long long)r * num_tiles;
  float m = -INFINITY;
  for (int j = 0; j < num_tiles; ++j) m = fmaxf(m, pm[j]);
  float s = 0.f;
  for (int j = 0; j < num_tiles; ++j) s += ps[j] * expf(pm[j] - m);
  float lse = m + logf(s);
  if (lse_out && DZ_STORE_OK(lse_out + r, 4)) lse_out[r] = lse;
  if (logprob && DZ_STORE_OK(logprob + r, 4)) logprob[r] = tgt_logit[r] - lse;
}

// One block.  mode 0: classification over candidates; mode 1: token-level CE.
__global__ void __launch_bounds__(256)
option_ce_kernel(const float* __restrict__ logprob, const int* __restrict__ seq_start, int n_seq,
                 const int* __restrict__ ex_start, const int* __restrict__ labels, int n_ex, int mode,
                 float* __restrict__ seq_lp, float* __restrict__ loss_out) {
  __shared__ float s_red[256];
  float acc = 0.f;
  if (mode == 1) {
    int rows = seq_start[n_seq];
    for (int r = threadIdx.x; r < rows; r += blockDim.x) acc -= logprob[r];
    s_red[threadIdx.x] = acc;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
      if (threadIdx.x < s) s_red[threadIdx.x] += s_red[threadIdx.x + s];
      __syncthreads();
    }
    if (threadIdx.x == 0) loss_out[0] = rows > 0 ? s_red[0] / rows : 0.f;
    return;
  }
  for (int s = threadIdx.x; s < n_seq; s += blockDim.x) {
    int r0 = seq_start[s], r1 = seq_start[s + 1];
    float t = 0.f;
    for (int r = r0; r < r1; ++r) t += logprob[r];
    seq_lp[s] = r1 > r0 ? t / (r1 - r0) : 0.f;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_ex; e += blockDim.x) {
    int c0 = ex_start[e], c1 = ex_start[e + 1];
    float m = -INFINITY;
    for (int c = c0; c < c1; ++c) m = fmaxf(m, seq_lp[c]);
    float s = 0.f;
    for (int c = c0; c < c1; ++c) s += expf(seq_lp[c] - m);
    acc += (m + logf(s)) - seq_lp[c0 + labels[e]];
  }
  s_red[threadIdx.x] = acc;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) s_red[threadIdx.x] += s_red[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) loss_out[0] = n_ex > 0 ? s_red[0] / n_ex : 0.f;
}

// One block of 256 threads: logits[e, c] = <h[e], table[cand[c]]>, loss = mean_e CE.
__global__ void __launch_bounds__(256)
verbalizer_ce_kernel(const __nv_bfloat16* __restrict__ h, long long ldh,
                     const __nv_bfloat16* __restrict__ table, long long ldt,
                     const int* __restrict__ cand, int n_cand, const int* __restrict__ labels,
                     int n_ex, int d, float* __restrict__ logits, float* __restrict__ loss_out) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarp = blockDim.x >> 5;
  for (int pair = warp; pair < n_ex * n_cand; pair += nwarp) {
    int e = pair / n_cand, c = pair - e * n_cand;
    const uint4* hr = reinterpret_cast<const uint4*>(h + (long long)e * ldh);
    const uint4* tr = reinterpret_cast<const uint4*>(table + (long long)cand[c] * ldt);
    float acc = 0.f;
    for (int i = lane; i < (d >> 3); i += 32) {
      uint4 a = hr[i], b = __ldg(tr + i);
      acc = fmaf(bf16_lo(a.x), bf16_lo(b.x), acc); acc = fmaf(bf16_hi(a.x), bf16_hi(b.x), acc);
      acc = fmaf(bf16_lo(a.y), bf16_lo(b.y), acc); acc = fmaf(bf16_hi(a.y), bf16_hi(b.y), acc);
      acc = fmaf(bf16_lo(a.z), bf16_lo(b.z), acc); acc = fmaf(bf16_hi(a.z), bf16_hi(b.z), acc);
      acc = fmaf(bf16_lo(a.w), bf16_lo(b.w), acc); acc = fmaf(bf16_hi(a.w), bf16_hi(b.w), acc);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) logits[pair] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0 && loss_out) {
    float tot = 0.f;
    for (int e = 0; e < n_ex; ++e) {
      const float* lg = logits + e * n_cand;
      float m = -INFINITY;
      for (int c = 0; c < n_cand; ++c) m = fmaxf(m, lg[c]);
      float s = 0.f;
      for (int c = 0; c < n_cand; ++c) s += expf(lg[c] - m);
      tot += (m + logf(s)) - lg[labels[e]];
    }
    loss_out[0] = tot / n_ex;
  }
}

}  // namespace dz

using namespace dz;
DZ_DEBUG_TU(lmhead)

extern "C" int dz_lse_combine(const float* part_max, const float* part_sum, const float* tgt_logit,
                              int num_tiles, int rows, float* logprob, float* lse_out,
                              cudaStream_t stream) {
  if (!part_max || !part_sum || rows <= 0 || num_tiles <= 0) return DZ_ERR_ARG;
  if (logprob && !tgt_logit) return DZ_ERR_ARG;
  lse_combine_kernel<<<(rows + 127) / 128, 128, 0, stream>>>(part_max, part_sum, tgt_logit,
                                                             num_tiles, rows, logprob, lse_out);
  return cuda_rc(cudaGetLastError());
}

extern "C" int dz_option_ce(const float* logprob, const int* seq_start, int n_seq,
                            const int* ex_start, const int* labels, int n_ex, int mode,
                            float* seq_lp, float* loss_out, cudaStream_t stream) {
  if (!logprob || !seq_start || !loss_out || n_seq <= 0) return DZ_ERR_ARG;
  if (mode == 0 && (!ex_start || !labels || !seq_lp || n_ex <= 0)) return DZ_ERR_ARG;
  option_ce_kernel<<<1, 256, 0, stream>>>(logprob, seq_start, n_seq, ex_start, labels, n_ex, mode,
                                          seq_lp, loss_out);
  return cuda_rc(cudaGetLastError());
}

extern "C" int dz_verbalizer_ce(const void* h, long long ldh, const void* table, long long ldt,
                                const int* cand, int n_cand, const int* labels, int n_ex, int d,
                                float* logits, float* loss_out, cudaStream_t stream) {
  if (!h || !table || !cand || !logits || n_cand <= 0 || n_ex <= 0) return DZ_ERR_ARG;
  if (loss_out && !labels) return DZ_ERR_ARG;
  if ((d & 7) || (ldh & 7) || (ldt & 7) || (reinterpret_cast<uintptr_t>(h) & 15) ||
      (reinterpret_cast<uintptr_t>(table) & 15))
    return DZ_ERR_ALIGN;
  verbalizer_ce_kernel<<<1, 256, 0, stream>>>((const __nv_bfloat16*)h, ldh,
                                              (const __nv_bfloat16*)table, ldt, cand, n_cand, labels,
                                              n_ex, d, logits, loss_out);
  return cuda_rc(cudaGetLastError());
}
