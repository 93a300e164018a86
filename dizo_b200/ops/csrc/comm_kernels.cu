// Small collectives over peer memory (NVLink / NVSwitch), written as kernels so that the
// exchange and the arithmetic that consumes it are one launch.
//
// Peer buffers are symmetric allocations: every rank holds the same layout and knows every
// peer's base pointer.  Synchronisation uses monotonically increasing 32-bit epochs written
// with release semantics at system scope into the receiver's flag words and polled with
// acquire loads; every poll is bounded (DZ_WAIT_TIMEOUT_NS) and reports through the error word
// instead of spinning forever when a peer is missing.
//
//   dz_peer_barrier            : all ranks have reached this point of their streams
//   dz_norm_allreduce_gamma    : all-reduce (sum) of the per-tensor squared distances
//                                ||theta_i - theta_0i||^2 of sharded parameters + the gamma
//                                initialisation / alpha = gamma / (ts + 1e-8) of the DiZO
//                                projection, in one kernel (P2P stores, fixed summation order;
//                                optionally multimem.ld_reduce through NVSwitch)
//   dz_rs_reduce_layernorm     : the owner side of GEMM -> reduce-scatter: waits for every
//                                rank's partial tile rows, h = residual + bias + sum_r part_r
//                                (fixed order), y = LayerNorm(h)
// Reference call sites replaced: torch.norm per tensor (large_models/trainer.py:581-584) and
// the alpha arithmetic (:453-465) under sharding; the reference itself has no sharded ZO path.
#include "common.cuh"
#include "host_util.h"

namespace dz {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Wait until *p >= epoch (wrap-safe).  Returns false after the time limit.
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t epoch, uint32_t* err,
                                          uint32_t code) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while ((int32_t)(ld_acquire_sys(p) - epoch) < 0) {
    if ((++spins & 0x3f) == 0) {
      uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > DZ_WAIT_TIMEOUT_NS) {
        if (err) atomicCAS(err, 0u, code | (blockIdx.x << 8));
        return false;
      }
    }
    __nanosleep(64);
  }
  return true;
}

// flags: per rank [world] words; rank r writes `epoch` into word [r] of every peer's array.
__global__ void peer_barrier_kernel(uint32_t* const* flag_ptrs, int rank, int world, uint32_t epoch,
                                    uint32_t* err) {
  int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    st_release_sys(flag_ptrs[t] + rank, epoch);
    wait_flag(flag_ptrs[rank] + t, epoch, err, ERR_WAIT_PEER);
  }
}

// slots: per rank a [world][n] fp32 area; rank r writes its partial vector into slot [r] of
// every rank (its own included), raises flag word [r] there, waits for all, sums in rank order.
// mode bit0: also run the gamma initialisation (ts = sqrt(sq); gamma = ts if reinit);
// alpha = gamma / (ts + 1e-8) is always refreshed.
__global__ void norm_allreduce_gamma_kernel(const float* partial, int n, float* const* slot_ptrs,
                                            uint32_t* const* flag_ptrs, float* mc_local,
                                            const float* mc_addr, int rank, int world, uint32_t epoch, float* sq_out,
                                            float* ts, float* gamma, float* alpha, int reinit,
                                            int use_multimem, uint32_t* err) {
  __shared__ int s_ok;
  const int t = threadIdx.x;
  // 1. publish
  for (int i = t; i < n * world; i += blockDim.x) {
    int peer = i / n, j = i - peer * n;
    slot_ptrs[peer][(size_t)rank * n + j] = partial[j];
  }
  // NVSwitch path: the same offset of every rank's buffer holds that rank's partial
  if (use_multimem && mc_local)
    for (int j = t; j < n; j += blockDim.x) mc_local[j] = partial[j];
  __threadfence_system();
  __syncthreads();
  if (t == 0) s_ok = 1;
  __syncthreads();
  if (t < world) {
    st_release_sys(flag_ptrs[t] + rank, epoch);
    if (!wait_flag(flag_ptrs[rank] + t, epoch, err, ERR_WAIT_PEER)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  // 2. reduce (fixed order) + gamma arithmetic
  const float* mine = slot_ptrs[rank];
  for (int j = t; j < n; j += blockDim.x) {
    float s = 0.f;
    if (use_multimem && mc_addr) {
      // one load through the multicast address sums the world copies inside the switch
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.f32 %0, [%1];"
                   : "=f"(s)
                   : "l"(mc_addr + j)
                   : "memory");
    } else {
      for (int r = 0; r < world; ++r) s += mine[(size_t)r * n + j];
    }
    sq_out[j] = s;
    float tsv = sqrtf(s);
    ts[j] = tsv;
    float g = reinit ? tsv : gamma[j];
    gamma[j] = g;
    alpha[j] = g / (tsv + 1e-8f);
  }
}

constexpr int RSLN_MAXV = 4;

// Owner side of GEMM -> reduce-scatter.  part: [world][rows][ld_part] bf16 (slot r written by
// rank r's GEMM epilogue over NVLink); flags[r] >= epoch once rank r has finished writing.
// Pull form (mc_part != nullptr, flags == nullptr, world == 0): every rank kept its whole partial
// product in its own copy of one symmetric buffer and a peer barrier ran since; mc_part is the
// NVSwitch multicast address of this rank's first row there, and one multimem.ld_reduce per 16
// bytes returns the sum over the ranks (added in fp32 inside the switch, rounded to bf16 once).
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
rs_reduce_layernorm_kernel(const __nv_bfloat16* __restrict__ part, long long slot_stride,
                           long long ld_part, const uint32_t* flags, uint32_t epoch, int world,
                           const __nv_bfloat16* __restrict__ residual, long long ldr,
                           const __nv_bfloat16* __restrict__ bias,
                           const __nv_bfloat16* __restrict__ lnw, const __nv_bfloat16* __restrict__ lnb,
                           __nv_bfloat16* __restrict__ h_out, long long ldh,
                           __nv_bfloat16* __restrict__ y_out, long long ldy, int d, float eps,
                           uint32_t* err, const __nv_bfloat16* mc_part) {
  __shared__ float s_red[THREADS / 32];
  __shared__ float s_bcast;
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (flags && (int)threadIdx.x < world) {
    if (!wait_flag(flags + threadIdx.x, epoch, err, ERR_WAIT_PEER)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const long long row = blockIdx.x;
  const int nvec = d >> 3;
  float v[RSLN_MAXV][8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < RSLN_MAXV; ++i) {
    int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      uint4 r4 = *reinterpret_cast<const uint4*>(residual + row * ldr + idx * 8);
      uint4 b4 = bias ? __ldg(reinterpret_cast<const uint4*>(bias) + idx) : make_uint4(0, 0, 0, 0);
      const uint32_t rr[4] = {r4.x, r4.y, r4.z, r4.w}, bb[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[i][2 * j] = bf16_lo(rr[j]) + bf16_lo(bb[j]);
        v[i][2 * j + 1] = bf16_hi(rr[j]) + bf16_hi(bb[j]);
      }
      if (mc_part) {
        uint4 p4;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(p4.x), "=r"(p4.y), "=r"(p4.z), "=r"(p4.w)
                     : "l"(mc_part + row * ld_part + idx * 8));
        const uint32_t pp[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[i][2 * j] += bf16_lo(pp[j]);
          v[i][2 * j + 1] += bf16_hi(pp[j]);
        }
      }
      for (int r = 0; r < world; ++r) {
        uint4 p4 = *reinterpret_cast<const uint4*>(part + r * slot_stride + row * ld_part + idx * 8);
        const uint32_t pp[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[i][2 * j] += bf16_lo(pp[j]);
          v[i][2 * j + 1] += bf16_hi(pp[j]);
        }
      }
      uint4 o;
      o.x = pack_bf16x2(v[i][0], v[i][1]); o.y = pack_bf16x2(v[i][2], v[i][3]);
      o.z = pack_bf16x2(v[i][4], v[i][5]); o.w = pack_bf16x2(v[i][6], v[i][7]);
      *reinterpret_cast<uint4*>(h_out + row * ldh + idx * 8) = o;
      // normalise what was stored (the bf16 residual stream), like the unsharded path
      const uint32_t oo[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[i][2 * j] = bf16_lo(oo[j]);
        v[i][2 * j + 1] = bf16_hi(oo[j]);
        sum += v[i][2 * j] + v[i][2 * j + 1];
      }
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
  if (!y_out) return;
  const float mean = block_sum(sum) / d;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < RSLN_MAXV; ++i) {
    int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float dl = v[i][j] - mean;
        sq = fmaf(dl, dl, sq);
      }
    }
  }
  const float rstd = rsqrtf(block_sum(sq) / d + eps);
#pragma unroll
  for (int i = 0; i < RSLN_MAXV; ++i) {
    int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      uint4 w4 = __ldg(reinterpret_cast<const uint4*>(lnw) + idx);
      uint4 b4 = __ldg(reinterpret_cast<const uint4*>(lnb) + idx);
      const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w}, bb[4] = {b4.x, b4.y, b4.z, b4.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[j] = pack_bf16x2((v[i][2 * j] - mean) * rstd * bf16_lo(ww[j]) + bf16_lo(bb[j]),
                           (v[i][2 * j + 1] - mean) * rstd * bf16_hi(ww[j]) + bf16_hi(bb[j]));
      *reinterpret_cast<uint4*>(y_out + row * ldy + idx * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

}  // namespace dz

using namespace dz;

extern "C" int dz_peer_barrier(const void* flag_ptrs_dev, int rank, int world, uint32_t epoch,
                               uint32_t* err, cudaStream_t stream) {
  if (!flag_ptrs_dev || world <= 0 || world > 32 || rank < 0 || rank >= world) return DZ_ERR_ARG;
  peer_barrier_kernel<<<1, 32, 0, stream>>>((uint32_t* const*)flag_ptrs_dev, rank, world, epoch, err);
  return cuda_rc(cudaGetLastError());
}

extern "C" int dz_norm_allreduce_gamma(const float* partial, int n, const void* slot_ptrs_dev,
                                       const void* flag_ptrs_dev, float* mc_local,
                                       const float* mc_addr, int rank, int world, uint32_t epoch, float* sq_out, float* ts,
                                       float* gamma, float* alpha, int reinit, int use_multimem,
                                       uint32_t* err, cudaStream_t stream) {
  if (!partial || !slot_ptrs_dev || !flag_ptrs_dev || !sq_out || !ts || !gamma || !alpha) return DZ_ERR_ARG;
  if (n <= 0 || world <= 0 || world > 32 || rank < 0 || rank >= world) return DZ_ERR_ARG;
  norm_allreduce_gamma_kernel<<<1, 256, 0, stream>>>(partial, n, (float* const*)slot_ptrs_dev,
                                                     (uint32_t* const*)flag_ptrs_dev, mc_local, mc_addr,
                                                     rank, world, epoch, sq_out, ts, gamma, alpha, reinit,
                                                     use_multimem, err);
  return cuda_rc(cudaGetLastError());
}

static int rs_reduce_layernorm_launch(const void* part, long long slot_stride, long long ld_part,
                                      const uint32_t* flags, uint32_t epoch, int world,
                                      const void* residual, long long ldr, const void* bias,
                                      const void* lnw, const void* lnb, void* h_out, long long ldh,
                                      void* y_out, long long ldy, long long rows, int d, float eps,
                                      uint32_t* err, const void* mc_rows, cudaStream_t stream);

extern "C" int dz_rs_reduce_layernorm(const void* part, long long slot_stride, long long ld_part,
                                      const uint32_t* flags, uint32_t epoch, int world,
                                      const void* residual, long long ldr, const void* bias,
                                      const void* lnw, const void* lnb, void* h_out, long long ldh,
                                      void* y_out, long long ldy, long long rows, int d, float eps,
                                      uint32_t* err, cudaStream_t stream) {
  return rs_reduce_layernorm_launch(part, slot_stride, ld_part, flags, epoch, world, residual, ldr, bias, lnw,
                                    lnb, h_out, ldh, y_out, ldy, rows, d, eps, err, nullptr, stream);
}

// Pull form of the above: mc_rows = multicast address of this rank's first row of the symmetric
// partial-product buffer (row pitch ld_part); the caller ran a peer barrier after its GEMM.
extern "C" int dz_rs_pull_layernorm(const void* mc_rows, long long ld_part, const void* residual,
                                    long long ldr, const void* bias, const void* lnw, const void* lnb,
                                    void* h_out, long long ldh, void* y_out, long long ldy,
                                    long long rows, int d, float eps, uint32_t* err, cudaStream_t stream) {
  if (!mc_rows || ((uintptr_t)mc_rows & 15)) return DZ_ERR_ALIGN;
  return rs_reduce_layernorm_launch(nullptr, 0, ld_part, nullptr, 0, 0, residual, ldr, bias, lnw, lnb, h_out,
                                    ldh, y_out, ldy, rows, d, eps, err, mc_rows, stream);
}

static int rs_reduce_layernorm_launch(const void* part, long long slot_stride, long long ld_part,
                                      const uint32_t* flags, uint32_t epoch, int world,
                                      const void* residual, long long ldr, const void* bias,
                                      const void* lnw, const void* lnb, void* h_out, long long ldh,
                                      void* y_out, long long ldy, long long rows, int d, float eps,
                                      uint32_t* err, const void* mc_rows, cudaStream_t stream) {
  if (!mc_rows && (!part || !flags || world <= 0)) return DZ_ERR_ARG;
  if (!residual || !h_out || rows <= 0 || d <= 0 || world < 0 || world > 32)
    return DZ_ERR_ARG;
  if (y_out && (!lnw || !lnb)) return DZ_ERR_ARG;
  if ((d & 7) || (ld_part & 7) || (ldr & 7) || (ldh & 7) || (slot_stride & 7) || (y_out && (ldy & 7)))
    return DZ_ERR_ALIGN;
  const int nvec = d >> 3;
  auto P = (const __nv_bfloat16*)part; auto R = (const __nv_bfloat16*)residual;
  auto B = (const __nv_bfloat16*)bias; auto W = (const __nv_bfloat16*)lnw; auto Lb = (const __nv_bfloat16*)lnb;
  auto H = (__nv_bfloat16*)h_out; auto Y = (__nv_bfloat16*)y_out;
  auto MC = (const __nv_bfloat16*)mc_rows;
  if (nvec <= 128 * RSLN_MAXV)
    rs_reduce_layernorm_kernel<128><<<(unsigned)rows, 128, 0, stream>>>(P, slot_stride, ld_part, flags, epoch, world, R, ldr, B, W, Lb, H, ldh, Y, ldy, d, eps, err, MC);
  else if (nvec <= 256 * RSLN_MAXV)
    rs_reduce_layernorm_kernel<256><<<(unsigned)rows, 256, 0, stream>>>(P, slot_stride, ld_part, flags, epoch, world, R, ldr, B, W, Lb, H, ldh, Y, ldy, d, eps, err, MC);
  else if (nvec <= 512 * RSLN_MAXV)
    rs_reduce_layernorm_kernel<512><<<(unsigned)rows, 512, 0, stream>>>(P, slot_stride, ld_part, flags, epoch, world, R, ldr, B, W, Lb, H, ldh, Y, ldy, d, eps, err, MC);
  else
    return DZ_ERR_TOO_LARGE;
  return cuda_rc(cudaGetLastError());
}
