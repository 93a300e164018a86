// Zeroth-order parameter sweeps over a flat bf16 parameter arena.
//
// All trainable tensors of a model live in one bf16 buffer.  A table describes them:
// {offset, numel, tensor id (RNG stream), DiZO slot or -1, offset of the anchor copy}.
// Tensor starts are aligned to ZO_CHUNK (256) elements, so every 256-element chunk (one
// warp x 16 bytes per lane) belongs to exactly one tensor, and one launch sweeps any
// contiguous range of the arena (one layer, or the whole model).  256 divides every OPT
// hidden size, so q/k/v weights (and biases) packed back to back stay contiguous and can
// be read as one fused [3d, d] operand.
//
// dz_zo_sweep computes, per element of every tensor in the range,
//     v   = theta                                   (bf16 -> fp32)
//     v   = anchor + alpha[slot] * (v - anchor)     if BLEND and the tensor has a slot
//     v  += c1 * z(seed1) + c2 * z(seed2)           z regenerated from Philox in registers
//     dst = bf16(v)                                 round-to-nearest or stochastic
// (fp32 arithmetic), except for the plain perturbation dst = theta + c1 z(seed1) - the sweep
// every forward pass runs - which stays in packed bf16: dst = fma.rn.bf16x2(bf16(c1), z, theta),
// exact product and sum with one rounding, and none of the unpack / convert / pack instructions.
//     chunk_sq[chunk] = sum (v - anchor)^2          if NORM and the tensor has a slot
// dst may be the arena itself (in-place perturb / restore / update / projection) or a
// staging buffer (perturbed or projected weights for one forward, theta untouched).
// Coefficients can come from device memory (c = coef_scale * *coef_ptr), so the
// projected gradient never visits the host between the two forwards and the update.
//
// Replaces the reference's per-tensor torch.normal + three elementwise passes
// (large_models/trainer.py:1438-1444), its update (:1603-1608), the per-tensor norms
// (:581-584) and the apply/reverse projection passes (:405-451).
#include "common.cuh"
#include "host_util.h"
#include "philox.cuh"

namespace dz {

constexpr int ZO_CHUNK = 256;    // elements; tensor starts are aligned to this (one warp pass)
constexpr int ZO_THREADS = 768;  // one persistent CTA (24 warps) per SM
constexpr int ZO_THREADS_SMALL = 512;  // the variant that shares an SM with a GEMM CTA
constexpr int ZO_SMEM_SMALL = GAUSS_BINS * 4;
constexpr int ZO_UNROLL = 4;     // 16-byte loads in flight per lane
constexpr int ZO_SMEM = GAUSS_SMEM_BYTES; // the lane-replicated inverse-CDF table

struct ZoTensor {
  long long offset;         // first element in the arena
  long long numel;
  long long anchor_offset;  // first element in the anchor arena (valid if slot >= 0)
  int tensor_id;            // RNG stream id, stable under any sharding
  int slot;                 // DiZO constraint index, or -1
  long long elem_base;      // index of this piece's first element inside the full tensor
  // Column-sharded pieces of a 2-D tensor (tensor parallel): the piece holds `local_cols`
  // of the `full_cols` columns of every row, starting at column `col0` (all multiples of
  // 8).  local_cols == 0 means the piece is contiguous inside the full tensor.
  long long local_cols, full_cols, col0;
  long long sq_base;        // index of this piece's first chunk in the norm partials, or -1
};

__device__ __forceinline__ uint32_t zo_group(const ZoTensor& t, long long e0) {
  long long ge = t.elem_base + e0;
  if (t.local_cols) {
    long long r = e0 / t.local_cols;
    ge = t.elem_base + r * t.full_cols + t.col0 + (e0 - r * t.local_cols);
  }
  return static_cast<uint32_t>(ge >> 3);
}

struct ZoSweepArgs {
  const __nv_bfloat16* src;     // arena
  __nv_bfloat16* dst;           // arena (in place) or staging laid out like the arena range
  __nv_bfloat16* dst2;          // optional second staging area: receives theta - c1 z while dst receives theta + c1 z
  long long dst_shift;          // dst element index = arena element index - dst_shift
  const __nv_bfloat16* anchor;  // anchor arena (theta_0 of the slotted tensors) or null
  const ZoTensor* table;
  int t_begin, t_end;           // tensors of the range
  long long chunk_begin, chunk_end;
  unsigned long long seed1, seed2;
  const unsigned long long* seed1_dev;   // if set: seed1 is read from the device (graph replays)
  float c1, c2;                 // host coefficients
  const float* c1_ptr;          // if set: c1 = c1 * *c1_ptr
  const float* c2_ptr;
  const float* alpha;           // [slots] blend ratios
  float* chunk_sq;              // norm partials: [sq_base + chunk inside the piece]
  unsigned long long sr_seed;   // stochastic rounding stream
  const uint32_t* gauss_table;  // [1024] (a', b) pairs of the inverse normal CDF (global memory)
};

__device__ __forceinline__ int find_tensor(const ZoTensor* tab, int lo, int hi, long long pos) {
  // last tensor in [lo, hi) whose offset <= pos
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (tab[mid].offset <= pos) lo = mid; else hi = mid;
  }
  return lo;
}

// One 256-element chunk: lane l owns elements [8l, 8l+8).  `raw` was loaded by the caller.
template <bool Z2, bool BLEND, bool NORM, bool SR, int TS>
__device__ __forceinline__ void zo_chunk(const ZoSweepArgs& a, const ZoTensor& t, float alpha,
                                         long long cpos, int lane, const uint4 raw,
                                         const char* tab, float c1, float c2, uint32_t c1_pair) {
  const long long e0 = cpos - t.offset + lane * 8;  // element inside this piece
  float sq = 0.f;
  constexpr bool PACKED = !Z2 && !BLEND && !NORM && !SR;
  if (PACKED) {
    if (e0 < t.numel) {
      uint4 o = raw, o2 = raw;
      if (c1 != 0.f) {
        if (a.dst2) perturb8_packed_dual<TS>(tab, a.seed1, t.tensor_id, zo_group(t, e0), c1_pair, raw, o, o2);
        else o = perturb8_packed<TS>(tab, a.seed1, t.tensor_id, zo_group(t, e0), c1_pair, raw);
      }
      if (e0 + 8 > t.numel) {
        // ragged tail of a tensor: keep the padding elements as they were
        uint32_t ov[4] = {o.x, o.y, o.z, o.w};
        uint32_t ov2[4] = {o2.x, o2.y, o2.z, o2.w};
        const uint32_t rawv[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (e0 + j >= t.numel) {
            const uint32_t m = (j & 1) ? 0xffff0000u : 0xffffu;
            ov[j >> 1] = (ov[j >> 1] & ~m) | (rawv[j >> 1] & m);
            ov2[j >> 1] = (ov2[j >> 1] & ~m) | (rawv[j >> 1] & m);
          }
        }
        o = make_uint4(ov[0], ov[1], ov[2], ov[3]);
        o2 = make_uint4(ov2[0], ov2[1], ov2[2], ov2[3]);
      }
      uint4* dp = reinterpret_cast<uint4*>(a.dst + (cpos + lane * 8 - a.dst_shift));
      if (DZ_STORE_OK(dp, 16)) *dp = o;
      if (a.dst2) {
        uint4* dp2 = reinterpret_cast<uint4*>(a.dst2 + (cpos + lane * 8 - a.dst_shift));
        if (DZ_STORE_OK(dp2, 16)) *dp2 = o2;
      }
    }
    return;
  }
  if (e0 < t.numel) {
    const long long pos = cpos + lane * 8;
    float v[8] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y),
                  bf16_lo(raw.z), bf16_hi(raw.z), bf16_lo(raw.w), bf16_hi(raw.w)};
    float an[8];
    const bool slotted = (BLEND || NORM) && t.slot >= 0;
    if (slotted) {
      uint4 ar = *reinterpret_cast<const uint4*>(a.anchor + t.anchor_offset + e0);
      an[0] = bf16_lo(ar.x); an[1] = bf16_hi(ar.x); an[2] = bf16_lo(ar.y); an[3] = bf16_hi(ar.y);
      an[4] = bf16_lo(ar.z); an[5] = bf16_hi(ar.z); an[6] = bf16_lo(ar.w); an[7] = bf16_hi(ar.w);
    }
    if (BLEND && slotted) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = fmaf(alpha, v[j] - an[j], an[j]);
    }
    const uint32_t grp = zo_group(t, e0);
    if (c1 != 0.f) {
      float z[8];
      gauss8<TS>(tab, a.seed1, t.tensor_id, grp, 0u, z);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = fmaf(c1, z[j], v[j]);
    }
    if (Z2) {
      float z[8];
      gauss8<TS>(tab, a.seed2, t.tensor_id, grp, 0u, z);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = fmaf(c2, z[j], v[j]);
    }
    uint32_t o[4];
    if (SR) {
      // stochastic rounding: add 16 random bits below the bf16 mantissa, truncate
      Philox4 rb = philox4x32<Z_PHILOX_ROUNDS>(grp, t.tensor_id, 1u, 0u, static_cast<uint32_t>(a.sr_seed),
                                  static_cast<uint32_t>(a.sr_seed >> 32));
      uint32_t rw[4] = {rb.x, rb.y, rb.z, rb.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t lo = __float_as_uint(v[2 * j]) + (rw[j] & 0xffffu);
        uint32_t hi = __float_as_uint(v[2 * j + 1]) + (rw[j] >> 16);
        o[j] = (lo >> 16) | (hi & 0xffff0000u);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
    }
    if (e0 + 8 > t.numel) {
      // ragged tail of a tensor: keep the padding elements as they were
      const uint32_t rawv[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (e0 + j >= t.numel) {
          uint32_t keep = (j & 1) ? (rawv[j >> 1] & 0xffff0000u) : (rawv[j >> 1] & 0xffffu);
          o[j >> 1] = (j & 1) ? ((o[j >> 1] & 0xffffu) | keep) : ((o[j >> 1] & 0xffff0000u) | keep);
        }
      }
    }
    uint4* dp = reinterpret_cast<uint4*>(a.dst + (pos - a.dst_shift));
    if (DZ_STORE_OK(dp, 16)) *dp = make_uint4(o[0], o[1], o[2], o[3]);
    if (NORM && slotted) {
      // norm of what was stored (the bf16 values), so it equals a later re-read
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (e0 + j < t.numel) {
          float w = (j & 1) ? bf16_hi(o[j >> 1]) : bf16_lo(o[j >> 1]);
          float d = w - an[j];
          sq = fmaf(d, d, sq);
        }
      }
    }
  }
  if (NORM) {
    // fixed-order warp reduction -> one partial per chunk (deterministic)
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
    if (lane == 0 && t.sq_base >= 0) {
      float* sp = a.chunk_sq + t.sq_base + (cpos - t.offset) / ZO_CHUNK;
      if (DZ_STORE_OK(sp, 4)) *sp = sq;
    }
  }
}

// Persistent: one CTA of 24 warps per SM.  The inverse-CDF table sits in shared memory (replicated per
// lane, conflict-free); every warp owns a contiguous run of chunks and works on ZO_UNROLL chunks at a
// time while the loads of the next ZO_UNROLL chunks are already in flight (register double buffering:
// 2 x 64 bytes per lane, ~100 KB per SM), so HBM latency is covered while z is computed.
//
// SMALL: the variant that runs beside a GEMM.  Its table is the plain 4 KB copy (bank conflicts
// instead of 128 KB of shared memory) and it is bounded to 512 threads x 64 registers, so one of its
// CTAs fits on an SM that already holds a GEMM CTA (~200 KB of shared memory, 192 threads): launched on
// a second stream it sweeps the next layer in the shadow of the tensor-core work, which leaves the
// issue slots and HBM almost idle.
template <bool Z2, bool BLEND, bool NORM, bool SR, bool SMALL>
__global__ void __launch_bounds__(SMALL ? ZO_THREADS_SMALL : ZO_THREADS, SMALL ? 2 : 1)
zo_sweep_kernel(const ZoSweepArgs a_in) {
  constexpr int THREADS = SMALL ? ZO_THREADS_SMALL : ZO_THREADS;
  constexpr int TS = SMALL ? 2 : 7;                 // log2 bytes between table entries
  ZoSweepArgs a = a_in;
  if (a.seed1_dev) {
    a.seed1 = *a.seed1_dev;     // a captured launch takes the step's seed from memory,
    if (SR) a.sr_seed = a.seed1 * 0x9E3779B97F4A7C15ull + 1ull;   // and its rounding stream follows the seed
  }
  extern __shared__ __align__(16) uint8_t zo_smem[];
  const char* tab;
  if (SMALL) {
    for (int i = threadIdx.x; i < GAUSS_BINS; i += THREADS)
      reinterpret_cast<uint32_t*>(zo_smem)[i] = __ldg(a.gauss_table + i);
    tab = reinterpret_cast<const char*>(zo_smem);
  } else {
    gauss_table_to_smem(zo_smem, a.gauss_table, threadIdx.x, THREADS);
    tab = reinterpret_cast<const char*>(zo_smem) + 4 * (threadIdx.x & 31);   // this lane's bank
  }
  __syncthreads();
  float c1 = a.c1, c2 = a.c2;
  if (a.c1_ptr) c1 *= __ldg(a.c1_ptr);
  if (Z2 && a.c2_ptr) c2 *= __ldg(a.c2_ptr);
  const uint32_t c1_pair = bf16x2_splat(c1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int WARPS = THREADS / 32;
  const long long total = a.chunk_end - a.chunk_begin;
  const long long nwarps = (long long)gridDim.x * WARPS;
  const long long per = (total + nwarps - 1) / nwarps;
  long long chunk = a.chunk_begin + ((long long)blockIdx.x * WARPS + warp) * per;
  const long long chunk_stop = min(chunk + per, a.chunk_end);
  if (chunk >= chunk_stop) return;

  int cur = find_tensor(a.table, a.t_begin, a.t_end, chunk * ZO_CHUNK);
  ZoTensor t = a.table[cur];
  long long t_next = (cur + 1 < a.t_end) ? a.table[cur + 1].offset : (1ll << 62);
  float alpha = 1.f;
  if (BLEND && t.slot >= 0) alpha = __ldg(a.alpha + t.slot);

  uint4 nxt[ZO_UNROLL];
  bool have = false;           // nxt holds the chunks [chunk, chunk + ZO_UNROLL)
  while (chunk < chunk_stop) {
    const long long cpos = chunk * ZO_CHUNK;
    if (cpos >= t_next) {
      ++cur;
      while (cur + 1 < a.t_end && a.table[cur + 1].offset <= cpos) ++cur;
      t = a.table[cur];
      t_next = (cur + 1 < a.t_end) ? a.table[cur + 1].offset : (1ll << 62);
      if (BLEND && t.slot >= 0) alpha = __ldg(a.alpha + t.slot);
    }
    // ZO_UNROLL full chunks of this tensor, inside this warp's run, start at chunk c
    const long long full_end = t.offset + (t.numel / ZO_CHUNK) * ZO_CHUNK;
    const bool fast = chunk + ZO_UNROLL <= chunk_stop && cpos + ZO_UNROLL * ZO_CHUNK <= full_end;
    if (fast) {
      uint4 raw[ZO_UNROLL];
#pragma unroll
      for (int u = 0; u < ZO_UNROLL; ++u)
        raw[u] = have ? nxt[u] : *reinterpret_cast<const uint4*>(a.src + cpos + u * ZO_CHUNK + lane * 8);
      const long long npos = cpos + ZO_UNROLL * ZO_CHUNK;
      // (the small variant has time to spare and registers to save: it does not prefetch)
      have = !SMALL && chunk + 2 * ZO_UNROLL <= chunk_stop && npos + ZO_UNROLL * ZO_CHUNK <= full_end;
      if (have) {
#pragma unroll
        for (int u = 0; u < ZO_UNROLL; ++u)
          nxt[u] = *reinterpret_cast<const uint4*>(a.src + npos + u * ZO_CHUNK + lane * 8);
      }
#pragma unroll
      for (int u = 0; u < ZO_UNROLL; ++u)
        zo_chunk<Z2, BLEND, NORM, SR, TS>(a, t, alpha, cpos + u * ZO_CHUNK, lane, raw[u], tab, c1, c2, c1_pair);
      chunk += ZO_UNROLL;
    } else {
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (cpos - t.offset + lane * 8 < t.numel)
        raw = *reinterpret_cast<const uint4*>(a.src + cpos + lane * 8);
      zo_chunk<Z2, BLEND, NORM, SR, TS>(a, t, alpha, cpos, lane, raw, tab, c1, c2, c1_pair);
      chunk += 1;
      have = false;
    }
  }
}

// Sum the per-chunk partials of each slotted tensor in fixed order: sq[slot] = sum.
__global__ void zo_reduce_chunks_kernel(const ZoTensor* table, int num_tensors,
                                        const float* chunk_sq, float* sq_out) {
  __shared__ float s_red[256];
  const int ti = blockIdx.x;
  if (ti >= num_tensors) return;
  const ZoTensor t = table[ti];
  if (t.slot < 0) return;
  const long long c0 = t.sq_base;
  const long long nchunks = (t.numel + ZO_CHUNK - 1) / ZO_CHUNK;
  float acc = 0.f;
  for (long long c = threadIdx.x; c < nchunks; c += blockDim.x) acc += chunk_sq[c0 + c];
  s_red[threadIdx.x] = acc;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) s_red[threadIdx.x] += s_red[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0 && DZ_STORE_OK(sq_out + t.slot, 4)) sq_out[t.slot] = s_red[0];  // one piece per slot per rank
}

// gamma search bookkeeping on the device (one thread per constraint).
//  mode 0 (init):    ts = sqrt(sq); gamma = ts (if reinit);
//  mode 1 (perturb): z = clip(N(0,1), +-(tau/eps) ts); gamma += delta*eps*z
//  mode 2 (step):    g = (*loss1 - *loss2)/(2 eps); gamma = clip(gamma - step*ts*g*z, (1-tau)ts, (1+tau)ts)
//  every mode then writes alpha = gamma / (ts + 1e-8).
// Matches large_models/trainer.py:545-562, :581-612, :453-465.
__global__ void gamma_step_kernel(int n, int mode, const float* sq, float* ts, float* gamma,
                                  float* zbuf, float* alpha, unsigned long long seed, int iter,
                                  float delta, float tau, float eps, float step_size,
                                  const float* loss1, const float* loss2, int reinit,
                                  const uint32_t* gauss_table) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float t;
  if (mode == 0) {
    t = sqrtf(sq[i]);
    ts[i] = t;
    if (reinit) gamma[i] = t;
  } else {
    t = ts[i];
  }
  float g = gamma[i];
  if (mode == 1) {
    float z;
    if (delta == 1.0f && iter >= 0) {
      Philox4 p = philox4x32<10>(static_cast<uint32_t>(i), static_cast<uint32_t>(iter), 2u, 0u,
                                 static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
      float z0 = gauss_scalar(gauss_table, p.x);
      float lim = (tau / eps) * t;
      z = fminf(fmaxf(z0, -lim), lim);
      zbuf[i] = z;
    } else {
      z = zbuf[i];
    }
    g += delta * z * eps;
  } else if (mode == 2) {
    float grad = (loss1[0] - loss2[0]) / (2.f * eps);
    g = g - step_size * t * grad * zbuf[i];
    g = fminf(fmaxf(g, (1.f - tau) * t), (1.f + tau) * t);
  }
  gamma[i] = g;
  alpha[i] = g / (t + 1e-8f);
}

// out = (a - b) * scale, all device scalars: the projected gradient (L+ - L-)/(2 eps).
__global__ void scalar_diff_kernel(const float* a, const float* b, float scale, float* out) {
  out[0] = (a[0] - b[0]) * scale;
}

template <bool Z2, bool BLEND, bool NORM, bool SR, bool SMALL = false>
static int launch_sweep(const ZoSweepArgs& a, cudaStream_t stream) {
  long long chunks = a.chunk_end - a.chunk_begin;
  if (chunks <= 0) return DZ_OK;
  auto kern = zo_sweep_kernel<Z2, BLEND, NORM, SR, SMALL>;
  constexpr int threads = SMALL ? ZO_THREADS_SMALL : ZO_THREADS;
  constexpr int smem = SMALL ? ZO_SMEM_SMALL : ZO_SMEM;
  if (!SMALL) {
    static PerDeviceFlag configured;
    if (int rc_cfg = ensure_dyn_smem(configured, kern, smem)) return rc_cfg;
  }
  long long blocks = (chunks + threads / 32 - 1) / (threads / 32);
  int grid = (int)(blocks < sm_count() ? blocks : sm_count());
  kern<<<grid, threads, smem, stream>>>(a);
  return cuda_rc(cudaGetLastError());
}

}  // namespace dz

using namespace dz;
DZ_DEBUG_TU(zo)

extern "C" int dz_zo_chunk() { return ZO_CHUNK; }
extern "C" int dz_zo_tensor_struct_bytes() { return (int)sizeof(ZoTensor); }

// One sweep over arena chunks [chunk_begin, chunk_end) (tensors [t_begin, t_end) of the
// table).  flags: bit0 second z term, bit1 blend with anchor, bit2 emit norm partials,
// bit3 stochastic rounding, bit4 the small-footprint variant that can share SMs with a GEMM
// (plain perturbation or blend only).
// seed1_dev (optional): device word holding seed1, read by the kernel instead of the argument, so
// that a launch captured in a CUDA graph perturbs with a new seed at every replay.
extern "C" int dz_zo_sweep_seeded(const void* src, void* dst, long long dst_shift, const void* anchor,
                                  const void* table, int t_begin, int t_end, long long chunk_begin,
                                  long long chunk_end, unsigned long long seed1,
                                  const unsigned long long* seed1_dev, float c1,
                                  const float* c1_ptr, unsigned long long seed2, float c2,
                                  const float* c2_ptr, const float* alpha, float* chunk_sq,
                                  unsigned long long sr_seed, int flags, const void* gauss_table,
                                  cudaStream_t stream) {
  if (!src || !dst || !table || !gauss_table || t_end <= t_begin) return DZ_ERR_ARG;
  if (reinterpret_cast<uintptr_t>(gauss_table) & 15) return DZ_ERR_ALIGN;
  const bool z2 = flags & 1, blend = flags & 2, norm = flags & 4, sr = flags & 8, small = flags & 16;
  if ((blend || norm) && !anchor) return DZ_ERR_ARG;
  if (blend && !alpha) return DZ_ERR_ARG;
  if (norm && !chunk_sq) return DZ_ERR_ARG;
  ZoSweepArgs a{};
  a.src = (const __nv_bfloat16*)src; a.dst = (__nv_bfloat16*)dst; a.dst_shift = dst_shift;
  a.anchor = (const __nv_bfloat16*)anchor; a.table = (const ZoTensor*)table;
  a.t_begin = t_begin; a.t_end = t_end; a.chunk_begin = chunk_begin; a.chunk_end = chunk_end;
  a.seed1 = seed1; a.seed1_dev = seed1_dev; a.seed2 = seed2; a.c1 = c1; a.c2 = c2; a.c1_ptr = c1_ptr; a.c2_ptr = c2_ptr;
  a.alpha = alpha; a.chunk_sq = chunk_sq; a.sr_seed = sr_seed;
  a.gauss_table = (const uint32_t*)gauss_table;
  int key = (z2 ? 1 : 0) | (blend ? 2 : 0) | (norm ? 4 : 0) | (sr ? 8 : 0);
  if (small) {
    if (key == 0) return launch_sweep<false, false, false, false, true>(a, stream);
    if (key == 2) return launch_sweep<false, true, false, false, true>(a, stream);
    return DZ_ERR_ARG;
  }
  switch (key) {
#define DZ_CASE(K, A, B, C, D) case K: return launch_sweep<A, B, C, D>(a, stream);
    DZ_CASE(0, false, false, false, false) DZ_CASE(1, true, false, false, false)
    DZ_CASE(2, false, true, false, false)  DZ_CASE(3, true, true, false, false)
    DZ_CASE(4, false, false, true, false)  DZ_CASE(5, true, false, true, false)
    DZ_CASE(6, false, true, true, false)   DZ_CASE(7, true, true, true, false)
    DZ_CASE(8, false, false, false, true)  DZ_CASE(9, true, false, false, true)
    DZ_CASE(10, false, true, false, true)  DZ_CASE(11, true, true, false, true)
    DZ_CASE(12, false, false, true, true)  DZ_CASE(13, true, false, true, true)
    DZ_CASE(14, false, true, true, true)   DZ_CASE(15, true, true, true, true)
#undef DZ_CASE
  }
  return DZ_ERR_ARG;
}

extern "C" int dz_zo_sweep(const void* src, void* dst, long long dst_shift, const void* anchor,
                           const void* table, int t_begin, int t_end, long long chunk_begin,
                           long long chunk_end, unsigned long long seed1, float c1,
                           const float* c1_ptr, unsigned long long seed2, float c2,
                           const float* c2_ptr, const float* alpha, float* chunk_sq,
                           unsigned long long sr_seed, int flags, const void* gauss_table,
                           cudaStream_t stream) {
  return dz_zo_sweep_seeded(src, dst, dst_shift, anchor, table, t_begin, t_end, chunk_begin, chunk_end, seed1,
                            nullptr, c1, c1_ptr, seed2, c2, c2_ptr, alpha, chunk_sq, sr_seed, flags,
                            gauss_table, stream);
}

// The two-point estimate's two staged copies from one draw of z: dst_plus = theta + c1 z, dst_minus = theta - c1 z
// (both laid out like the arena range, same dst_shift).  Plain perturbation only (the packed bf16 path).
extern "C" int dz_zo_sweep_dual(const void* src, void* dst_plus, void* dst_minus, long long dst_shift,
                                const void* table, int t_begin, int t_end, long long chunk_begin,
                                long long chunk_end, unsigned long long seed1,
                                const unsigned long long* seed1_dev, float c1, const float* c1_ptr, int small,
                                const void* gauss_table, cudaStream_t stream) {
  if (!src || !dst_plus || !dst_minus || !table || !gauss_table || t_end <= t_begin) return DZ_ERR_ARG;
  if (reinterpret_cast<uintptr_t>(gauss_table) & 15) return DZ_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(dst_plus) & 15) || (reinterpret_cast<uintptr_t>(dst_minus) & 15)) return DZ_ERR_ALIGN;
  ZoSweepArgs a{};
  a.src = (const __nv_bfloat16*)src; a.dst = (__nv_bfloat16*)dst_plus; a.dst2 = (__nv_bfloat16*)dst_minus;
  a.dst_shift = dst_shift; a.table = (const ZoTensor*)table;
  a.t_begin = t_begin; a.t_end = t_end; a.chunk_begin = chunk_begin; a.chunk_end = chunk_end;
  a.seed1 = seed1; a.seed1_dev = seed1_dev; a.c1 = c1; a.c1_ptr = c1_ptr;
  a.gauss_table = (const uint32_t*)gauss_table;
  if (small) return launch_sweep<false, false, false, false, true>(a, stream);
  return launch_sweep<false, false, false, false>(a, stream);
}

extern "C" int dz_zo_reduce_chunks(const void* table, int num_tensors, const float* chunk_sq,
                                   float* sq_out, cudaStream_t stream) {
  if (!table || !chunk_sq || !sq_out || num_tensors <= 0) return DZ_ERR_ARG;
  zo_reduce_chunks_kernel<<<num_tensors, 256, 0, stream>>>((const ZoTensor*)table, num_tensors,
                                                           chunk_sq, sq_out);
  return cuda_rc(cudaGetLastError());
}

extern "C" int dz_gamma_step(int n, int mode, const float* sq, float* ts, float* gamma, float* zbuf,
                             float* alpha, unsigned long long seed, int iter, float delta, float tau,
                             float eps, float step_size, const float* loss1, const float* loss2,
                             int reinit, const void* gauss_table, cudaStream_t stream) {
  if (n <= 0 || !ts || !gamma || !zbuf || !alpha || !gauss_table) return DZ_ERR_ARG;
  gamma_step_kernel<<<(n + 127) / 128, 128, 0, stream>>>(n, mode, sq, ts, gamma, zbuf, alpha, seed,
                                                         iter, delta, tau, eps, step_size, loss1,
                                                         loss2, reinit, (const uint32_t*)gauss_table);
  return cuda_rc(cudaGetLastError());
}

extern "C" int dz_scalar_diff(const float* a, const float* b, float scale, float* out,
                              cudaStream_t stream) {
  if (!a || !b || !out) return DZ_ERR_ARG;
  scalar_diff_kernel<<<1, 1, 0, stream>>>(a, b, scale, out);
  return cuda_rc(cudaGetLastError());
}

// z itself (fp32), for tests and for the CPU oracle that consumes the framework's stream.
__global__ void zo_fill_z_kernel(float* out, long long numel, long long elem_base,
                                 unsigned long long seed, int tensor_id, const uint32_t* tab) {
  long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long e0 = g * 8;
  if (e0 >= numel) return;
  float z[8];
  gauss8<2>(reinterpret_cast<const char*>(tab), seed, tensor_id, (uint32_t)((elem_base + e0) >> 3), 0u, z);
  for (int j = 0; j < 8 && e0 + j < numel; ++j)
    if (DZ_STORE_OK(out + e0 + j, 4)) out[e0 + j] = z[j];
}
extern "C" int dz_zo_fill_z(float* out, long long numel, long long elem_base,
                            unsigned long long seed, int tensor_id, const void* gauss_table,
                            cudaStream_t stream) {
  if (!out || !gauss_table || numel <= 0 || (elem_base & 7)) return DZ_ERR_ARG;
  long long groups = (numel + 7) / 8;
  zo_fill_z_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, stream>>>(out, numel, elem_base, seed,
                                                                        tensor_id, (const uint32_t*)gauss_table);
  return cuda_rc(cudaGetLastError());
}
