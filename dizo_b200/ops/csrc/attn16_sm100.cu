// Causal self-attention forward for sm_100a, sixteen-softmax-warp variant of attn_sm100.cu (same
// interface, masking and TMEM plan; see that file for the algorithm and the reference citations:
// large_models/ht_opt.py:209-272, large_models/prefix.py:28-53).
//
// attn_sm100.cu gives every query row to one thread, which handles all 128 scores of a key block;
// the softmax arithmetic of the two tiles then runs on 8 warps and is latency-bound.  Here a row
// is shared by two threads (warps w and w+4 of a tile's eight warps share a TMEM lane quadrant and
// split the 128 columns), so 16 warps work on the exponentials:
//   warps 0-7  : softmax for tile 0     warps 8-15 : softmax for tile 1
//   warp 16    : TMEM allocation; lane 0 issues tcgen05.mma
//   warp 17    : lane 0 = TMA producer
// The two threads of a row agree on the running maximum through shared memory (double-buffered
// slots, per-pair progress words polled with a bounded wait - no hardware barrier that a failed
// partner could leave hanging).  Each warp writes its packed P over the first 32 of the 64 columns
// it has just read, so P of a block lives at TMEM columns [0,32) and [64,96) of the S region.
#include "common.cuh"
#include "host_util.h"
#include "attn_args.h"

namespace dz {
namespace a16 {

constexpr int A_BQ = 128;    // query rows per tile
constexpr int A_BKV = 128;   // keys per block
constexpr int A_THREADS = 576;
constexpr int A_KV_STAGES = 2;
constexpr float A_RESCALE_THRESHOLD = 8.0f;  // log2 units

template <int HDP>
struct AttnSmem {
  static constexpr int Q_TILE = A_BQ * HDP * 2;     // per query tile
  static constexpr int KV_TILE = A_BKV * HDP * 2;   // per K or V stage
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + 2 * Q_TILE;
  static constexpr int OFF_V = OFF_K + A_KV_STAGES * KV_TILE;
  static constexpr int USED = OFF_V + A_KV_STAGES * KV_TILE + 1024;
  // at least 120 KB so that two CTAs (each wanting all 512 TMEM columns) never share an SM
  static constexpr int TOTAL = USED < 120 * 1024 ? 120 * 1024 : USED;
};

template <int HDP>
__global__ void __launch_bounds__(A_THREADS, 1)
attn_fwd16_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                const __grid_constant__ CUtensorMap tmPK, const __grid_constant__ CUtensorMap tmPV,
                const AttnArgs p) {
  using S = AttnSmem<HDP>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_q;
  __shared__ __align__(8) uint64_t bar_k_full[A_KV_STAGES], bar_k_empty[A_KV_STAGES];
  __shared__ __align__(8) uint64_t bar_v_full[A_KV_STAGES], bar_v_empty[A_KV_STAGES];
  __shared__ __align__(8) uint64_t bar_s[2], bar_p[2], bar_pv[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile int s_abort;
  __shared__ float s_x[2][2][2][A_BQ];        // [tile][block parity][half][row]: half-row maxima / sums
  __shared__ volatile int s_prog[2][4][2];    // [tile][quadrant][half]: blocks whose value is published

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  // Heaviest (latest) query tiles first: they have the most key blocks under causality.
  const int pairs = (p.L + 2 * A_BQ - 1) / (2 * A_BQ);
  const int pair = pairs - 1 - blockIdx.x;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int pad = p.pad_left ? p.pad_left[b] : 0;
  const int hd = p.hd;
  const int has_prefix = p.n_prefix > 0 ? 1 : 0;

  // Tile t covers query rows [q0[t], q0[t] + 128).  Block range of keys: [jb, nb[t]).
  int q0[2], nb[2], nvb[2];
  q0[0] = pair * 2 * A_BQ;
  q0[1] = q0[0] + A_BQ;
  const int jb = min(pad, q0[0]) / A_BKV;  // first block that can hold a visible key
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    if (q0[t] < p.L) {
      int last_row = min(q0[t] + A_BQ, p.L) - 1;
      nb[t] = last_row / A_BKV + 1;
      nvb[t] = has_prefix + nb[t] - jb;
    } else {
      nb[t] = jb;
      nvb[t] = 0;  // tile does not exist
    }
  }
  const int nvb_max = max(nvb[0], nvb[1]);

  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(smem_u32(&bar_q), 1);
    for (int s = 0; s < A_KV_STAGES; ++s) {
      mbar_init(smem_u32(&bar_k_full[s]), 1);
      mbar_init(smem_u32(&bar_k_empty[s]), 1);
      mbar_init(smem_u32(&bar_v_full[s]), 1);
      mbar_init(smem_u32(&bar_v_empty[s]), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(smem_u32(&bar_s[t]), 1);
      mbar_init(smem_u32(&bar_p[t]), 8);
      mbar_init(smem_u32(&bar_pv[t]), 1);
    }
    for (int i = 0; i < 16; ++i) (&s_prog[0][0][0])[i] = 0;
    fence_mbar_init();
  }
  if (warp == 16) {
    tmem_alloc(smem_u32(&s_tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  // TMEM columns: S0/P0 [0,128) S1/P1 [128,256) O0 [256,256+HDP) O1 [384,384+HDP)
  const uint32_t tm_s[2] = {tmem_base + 0u, tmem_base + 128u};
  const uint32_t tm_o[2] = {tmem_base + 256u, tmem_base + 384u};

  if (warp == 17) {
    if (lane == 0 && nvb_max > 0) {
      // ---------------------------------------------- TMA producer (one thread)
      const int row_base = b * p.L;
      {
        int ntile = (nvb[1] > 0) ? 2 : 1;
        mbar_arrive_expect_tx(smem_u32(&bar_q), ntile * S::Q_TILE);
        for (int t = 0; t < ntile; ++t)
          for (int c = 0; c < HDP / 64; ++c)
            tma_load_2d(smem_base + S::OFF_Q + t * S::Q_TILE + c * (A_BQ * 128), &tmQ,
                        smem_u32(&bar_q), p.q_col0 + h * hd + c * 64, row_base + q0[t]);
      }
      for (int vb = 0; vb < nvb_max; ++vb) {
        const int st = vb % A_KV_STAGES;
        const uint32_t ph = (vb / A_KV_STAGES) & 1;
        const bool pre = has_prefix && vb == 0;
        const int krow = pre ? 0 : row_base + (jb + vb - has_prefix) * A_BKV;
        if (!mbar_wait(smem_u32(&bar_k_empty[st]), ph ^ 1, &s_abort, p.err, ERR_WAIT_EMPTY)) break;
        {
          uint32_t full = smem_u32(&bar_k_full[st]);
          mbar_arrive_expect_tx(full, S::KV_TILE);
          for (int c = 0; c < HDP / 64; ++c) {
            uint32_t dst = smem_base + S::OFF_K + st * S::KV_TILE + c * (A_BKV * 128);
            if (pre) tma_load_2d(dst, &tmPK, full, h * hd + c * 64, 0);
            else tma_load_2d(dst, &tmKV, full, p.k_col0 + h * hd + c * 64, krow);
          }
        }
        if (!mbar_wait(smem_u32(&bar_v_empty[st]), ph ^ 1, &s_abort, p.err, ERR_WAIT_EMPTY)) break;
        {
          uint32_t full = smem_u32(&bar_v_full[st]);
          mbar_arrive_expect_tx(full, S::KV_TILE);
          for (int c = 0; c < HDP / 64; ++c) {
            uint32_t dst = smem_base + S::OFF_V + st * S::KV_TILE + c * (A_BKV * 128);
            if (pre) tma_load_2d(dst, &tmPV, full, h * hd + c * 64, 0);
            else tma_load_2d(dst, &tmKV, full, p.v_col0 + h * hd + c * 64, krow);
          }
        }
      }
    }
  } else if (warp == 16) {
    if (lane == 0 && nvb_max > 0) {
      // ---------------------------------------------- MMA issuer (one thread)
      bool ok = true;
      const uint32_t idesc_s = umma_idesc_bf16(A_BQ, A_BKV, 0, 0);
      const uint32_t idesc_o = umma_idesc_bf16(A_BQ, (hd + 15) & ~15, 0, 1);  // V is MN-major
      const int k_steps = (hd + 15) / 16;
      auto issue_s = [&](int t, int vb) {
        int st = vb % A_KV_STAGES;
        uint32_t qa = smem_base + S::OFF_Q + t * S::Q_TILE;
        uint32_t ka = smem_base + S::OFF_K + st * S::KV_TILE;
        for (int kk = 0; kk < k_steps; ++kk) {
          uint64_t ad = umma_desc_k_sw128(qa + (kk >> 2) * (A_BQ * 128) + (kk & 3) * 32);
          uint64_t bd = umma_desc_k_sw128(ka + (kk >> 2) * (A_BKV * 128) + (kk & 3) * 32);
          umma_bf16_ss(tm_s[t], ad, bd, idesc_s, kk != 0);
        }
        umma_commit(smem_u32(&bar_s[t]));
      };
      auto issue_pv = [&](int t, int vb) {
        int st = vb % A_KV_STAGES;
        uint32_t va = smem_base + S::OFF_V + st * S::KV_TILE;
        for (int kk = 0; kk < A_BKV / 16; ++kk) {
          // A = P from TMEM: 16 keys = 8 packed 32-bit columns (keys 0-63 at columns [0,32), keys
          // 64-127 at [64,96)).  B = V, MN-major: 16 keys = two 8-row groups of 1024 bytes; 64-column
          // blocks of the head are A_BKV*128 bytes apart.
          uint64_t bd = umma_desc_mn_sw128(va + kk * 2048, A_BKV * 128, 1024);
          umma_bf16_ts(tm_o[t], tm_s[t] + (kk >> 2) * 64 + (kk & 3) * 8, bd, idesc_o, (vb | kk) != 0);
        }
        umma_commit(smem_u32(&bar_pv[t]));
      };
      ok = mbar_wait(smem_u32(&bar_q), 0, &s_abort, p.err, ERR_WAIT_FULL);
      if (ok) ok = mbar_wait(smem_u32(&bar_k_full[0]), 0, &s_abort, p.err, ERR_WAIT_FULL);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (nvb[t] > 0) issue_s(t, 0);
        umma_commit(smem_u32(&bar_k_empty[0]));
      }
      for (int vb = 0; vb < nvb_max && ok; ++vb) {
        const int st = vb % A_KV_STAGES;
        const uint32_t ph = (vb / A_KV_STAGES) & 1;
        ok = mbar_wait(smem_u32(&bar_v_full[st]), ph, &s_abort, p.err, ERR_WAIT_FULL);
        if (!ok) break;
        const bool more = vb + 1 < nvb_max;
        if (more) {
          const int st1 = (vb + 1) % A_KV_STAGES;
          ok = mbar_wait(smem_u32(&bar_k_full[st1]), ((vb + 1) / A_KV_STAGES) & 1, &s_abort, p.err,
                         ERR_WAIT_FULL);
          if (!ok) break;
        }
        for (int t = 0; t < 2 && ok; ++t) {
          if (vb < nvb[t]) {
            ok = mbar_wait(smem_u32(&bar_p[t]), vb & 1, &s_abort, p.err, ERR_WAIT_MISC);
            if (!ok) break;
            tc_fence_after();
            issue_pv(t, vb);
            if (vb + 1 < nvb[t]) issue_s(t, vb + 1);
          }
        }
        if (!ok) break;
        // every MMA that reads V[vb] and K[vb+1] has been issued: release the stages
        umma_commit(smem_u32(&bar_v_empty[st]));
        if (more) umma_commit(smem_u32(&bar_k_empty[(vb + 1) % A_KV_STAGES]));
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    const int t = warp >> 3;                 // query tile
    const int quad = warp & 3;               // TMEM lane quadrant
    const int half = (warp >> 2) & 1;        // which 64 keys of a block
    const int r = quad * 32 + lane;          // row inside the tile
    const int qi = q0[t] + r;                // query index inside the sequence
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    float m_used = -INFINITY, l_sum = 0.f;   // l_sum: this thread's 64-column share
    bool ok = true;
    int published = 0;                       // values this warp has published to its partner

    // hand `mine` to the partner thread of the row and take its value (bounded wait)
    auto exchange = [&](float mine, float& other) -> bool {
      const int slot = published & 1;
      s_x[t][slot][half][r] = mine;
      __syncwarp();
      if (lane == 0) {
        __threadfence_block();
        s_prog[t][quad][half] = published + 1;
      }
      const volatile int* theirs = &s_prog[t][quad][half ^ 1];
      uint64_t t0 = 0;
      uint32_t spins = 0;
      bool good = true;
      while (*theirs < published + 1) {
        if ((++spins & 0xff) == 0) {
          if (s_abort) { good = false; break; }
          const uint64_t now = global_timer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > DZ_WAIT_TIMEOUT_NS) {
            s_abort = 1;
            if (p.err) atomicCAS(p.err, 0u, (uint32_t)ERR_WAIT_MISC | (blockIdx.x << 8));
            good = false;
            break;
          }
        }
      }
      good = __all_sync(0xffffffffu, good);
      if (good) {
        __threadfence_block();
        other = s_x[t][slot][half ^ 1][r];
      }
      ++published;
      return good;
    };

    for (int vb = 0; vb < nvb[t] && ok; ++vb) {
      ok = mbar_wait(smem_u32(&bar_s[t]), vb & 1, &s_abort, p.err, ERR_WAIT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool is_prefix = has_prefix && vb == 0;
      const int kv0 = (jb + vb - has_prefix) * A_BKV;
      // blocks entirely below the diagonal and right of the padding need no mask (uniform)
      const bool need_mask = is_prefix || !(kv0 + A_BKV - 1 <= q0[t] && kv0 >= pad);
      auto visible = [&](int c) -> bool {       // c: column inside the block
        if (is_prefix) return c < p.n_prefix;
        int kv = kv0 + c;
        return (kv <= qi) && (kv >= pad || kv == qi) && (kv < p.L);
      };
      // ---- this thread's 64 scores of the block in registers
      uint32_t sv[64];
      tmem_ld_32x32(tm_s[t] + lane_off + half * 64, sv);
      tmem_ld_32x32(tm_s[t] + lane_off + half * 64 + 32, sv + 32);
      tmem_ld_wait();
      float bm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          if (!visible(half * 64 + c)) sv[c] = 0xff800000u;  // -inf
          bm[c & 3] = fmaxf(bm[c & 3], __uint_as_float(sv[c]));
        }
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) bm[c & 3] = fmaxf(bm[c & 3], __uint_as_float(sv[c]));
      }
      float bmax = fmaxf(fmaxf(bm[0], bm[1]), fmaxf(bm[2], bm[3]));
      float other = -INFINITY;
      ok = exchange(bmax, other);
      if (!ok) break;
      bmax = fmaxf(bmax, other) * p.scale_log2;   // scale > 0: max commutes with the scaling
      // lazily raised maximum (both threads of the row compute the same decision)
      float m_new = m_used;
      if (bmax > m_used + A_RESCALE_THRESHOLD || m_used == -INFINITY) m_new = fmaxf(m_used, bmax);
      const bool changed = (m_new != m_used);
      if (vb > 0) {
        // PV of the previous block must be complete before O is touched or P overwritten
        ok = mbar_wait(smem_u32(&bar_pv[t]), (vb - 1) & 1, &s_abort, p.err, ERR_WAIT_MISC);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, changed && m_used != -INFINITY)) {
          const float f = (changed && m_used != -INFINITY) ? exp2f(m_used - m_new) : 1.0f;
          for (int c0 = half * 16; c0 < hd; c0 += 32) {      // the two warps of a quadrant alternate
            uint32_t o[16];
            tmem_ld_32x16(tm_o[t] + lane_off + c0, o);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * f);
            tmem_st_32x16(tm_o[t] + lane_off + c0, o);
          }
          tmem_st_wait();
        }
      }
      if (changed) {
        if (m_used != -INFINITY) l_sum *= exp2f(m_used - m_new);
        m_used = m_new;
      }
      // ---- probabilities -> bf16 pairs -> TMEM, over the first 32 of this warp's 64 columns
      const float mref = (m_used == -INFINITY) ? 0.f : m_used;
      float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        float e0 = exp2f(fmaf(__uint_as_float(sv[c]), p.scale_log2, -mref));
        float e1 = exp2f(fmaf(__uint_as_float(sv[c + 1]), p.scale_log2, -mref));
        ps[(c >> 1) & 3] += e0 + e1;
        sv[c >> 1] = pack_bf16x2(e0, e1);
      }
      tmem_st_32x16(tm_s[t] + lane_off + half * 64, sv);
      tmem_st_32x16(tm_s[t] + lane_off + half * 64 + 16, sv + 16);
      l_sum += (ps[0] + ps[1]) + (ps[2] + ps[3]);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_p[t]));
    }
    // ---- epilogue: O / l -> bf16 -> global
    if (ok && nvb[t] > 0) {
      float l_other = 0.f;
      ok = exchange(l_sum, l_other);
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_pv[t]), (nvb[t] - 1) & 1, &s_abort, p.err,
                                                      ERR_WAIT_MISC));
      if (ok) {
        tc_fence_after();
        const float l_tot = l_sum + l_other;
        const float inv = l_tot > 0.f ? 1.0f / l_tot : 0.f;
        const bool row_ok = qi < p.L;
        if (p.lse && row_ok && half == 0)
          p.lse[((long long)b * p.H + h) * p.L + qi] = l_tot > 0.f ? m_used + log2f(l_tot) : 0.f;
        __nv_bfloat16* orow = p.out + ((long long)b * p.L + qi) * p.ld_out + h * hd;
        for (int c0 = half * 16; c0 < hd; c0 += 32) {
          uint32_t o[16];
          tmem_ld_32x16(tm_o[t] + lane_off + c0, o);
          tmem_ld_wait();
          if (row_ok) {
            uint4 w0, w1;
            w0.x = pack_bf16x2(__uint_as_float(o[0]) * inv, __uint_as_float(o[1]) * inv);
            w0.y = pack_bf16x2(__uint_as_float(o[2]) * inv, __uint_as_float(o[3]) * inv);
            w0.z = pack_bf16x2(__uint_as_float(o[4]) * inv, __uint_as_float(o[5]) * inv);
            w0.w = pack_bf16x2(__uint_as_float(o[6]) * inv, __uint_as_float(o[7]) * inv);
            w1.x = pack_bf16x2(__uint_as_float(o[8]) * inv, __uint_as_float(o[9]) * inv);
            w1.y = pack_bf16x2(__uint_as_float(o[10]) * inv, __uint_as_float(o[11]) * inv);
            w1.z = pack_bf16x2(__uint_as_float(o[12]) * inv, __uint_as_float(o[13]) * inv);
            w1.w = pack_bf16x2(__uint_as_float(o[14]) * inv, __uint_as_float(o[15]) * inv);
            *reinterpret_cast<uint4*>(orow + c0) = w0;
            *reinterpret_cast<uint4*>(orow + c0 + 8) = w1;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 16) {
    __syncwarp();
    if (s_abort) {
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int HDP>
static int launch_attn16(const CUtensorMap& tmQ, const CUtensorMap& tmKV, const CUtensorMap& tmPK,
                       const CUtensorMap& tmPV, const AttnArgs& a, cudaStream_t stream) {
  using S = AttnSmem<HDP>;
  auto kern = attn_fwd16_kernel<HDP>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return cuda_rc(e);
    configured = true;
  }
  int pairs = (a.L + 2 * A_BQ - 1) / (2 * A_BQ);
  dim3 grid(pairs, a.H, a.B);
  kern<<<grid, A_THREADS, S::TOTAL, stream>>>(tmQ, tmKV, tmPK, tmPV, a);
  return cuda_rc(cudaGetLastError());
}

}  // namespace a16

// Same contract as launch_attn of attn_sm100.cu; called by dz_attn_fwd_lse when the variant is selected.
int launch_attn16_hd(int hdp, const CUtensorMap& tmQ, const CUtensorMap& tmKV, const CUtensorMap& tmPK,
                     const CUtensorMap& tmPV, const AttnArgs& a, cudaStream_t stream) {
  if (hdp == 64) return a16::launch_attn16<64>(tmQ, tmKV, tmPK, tmPV, a, stream);
  return a16::launch_attn16<128>(tmQ, tmKV, tmPK, tmPV, a, stream);
}

}  // namespace dz
