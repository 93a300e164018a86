// Causal self-attention forward for sm_100a (tcgen05 + TMEM), reading Q, K and V in
// place from the fused QKV projection output [B*L, 3*d] and writing the context
// [B*L, d] in the layout out_proj consumes.  No [L, L] score or mask tensor exists.
//
// Masking is computed from indices: key j is visible to query i of sequence b iff
//   j <= i  and  (j >= pad_left[b]  or  j == i)
// i.e. causal attention over left-padded batches (padding queries see only themselves,
// which keeps them finite; nothing real ever attends to them).  An optional block of
// `n_prefix` learned key/value rows per layer is visible to every query (prefix tuning).
// Replaces the bmm / additive-mask / softmax / bmm chain of
// large_models/ht_opt.py:209-272 and the K/V concatenation of large_models/prefix.py:28-53.
//
// One CTA = two 128-row query tiles of one (batch, head), 9 warps:
//   warps 0-3 : softmax for tile 0 (one thread per query row)
//   warps 4-7 : softmax for tile 1
//   warp 8    : TMEM allocation; lane 0 issues tcgen05.mma
//   warp 9    : lane 0 = TMA producer (Q once, then the K and V rings)
// Per 128-key block: S_t = Q_t K^T (TMEM) -> softmax threads read S with tcgen05.ld and write
// P (bf16, two per 32-bit column) back into TMEM over the columns S occupied -> O_t += P V
// with P as the TMEM A operand of tcgen05.mma, accumulating in TMEM.  P never touches shared
// memory.  The running row maximum is only raised when it grows by more than 2^8 (then O is
// rescaled in TMEM), so most blocks need no correction pass; blocks entirely below the
// diagonal skip the mask arithmetic.  The two tiles ping-pong: the tensor core works on one
// tile while the other does its exps.
#include "common.cuh"
#include "host_util.h"
#include "attn_args.h"

namespace dz {

constexpr int A_BQ = 128;    // query rows per tile
constexpr int A_BKV = 128;   // keys per block
constexpr int A_THREADS = 320;
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
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
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
      mbar_init(smem_u32(&bar_p[t]), 4);
      mbar_init(smem_u32(&bar_pv[t]), 1);
    }
    fence_mbar_init();
  }
  if (warp == 8) {
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

  if (warp == 9) {
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
  } else if (warp == 8) {
    if (lane == 0 && nvb_max > 0) {
      // ---------------------------------------------- MMA issuer (one thread)
      bool ok = true;
      const uint32_t idesc_s = umma_idesc_bf16(A_BQ, A_BKV, 0, 0);
      const uint32_t idesc_o = umma_idesc_bf16(A_BQ, (hd + 15) & ~15, 0, 1);  // V is MN-major
      const int k_steps = (hd + 15) / 16;
      // One thread issues every MMA, and a 128 x 128 x 16 product occupies the tensor pipe for only 64 cycles:
      // the descriptors are built once and each MMA adds a constant to their address field, so that issuing
      // stays cheaper than executing (building them per MMA took about 90 cycles each).
      const uint64_t q_desc0 = umma_desc_k_sw128(smem_base + S::OFF_Q);
      const uint64_t q_desc1 = umma_desc_k_sw128(smem_base + S::OFF_Q + S::Q_TILE);
      const uint64_t k_desc0 = umma_desc_k_sw128(smem_base + S::OFF_K);
      const uint64_t k_desc1 = umma_desc_k_sw128(smem_base + S::OFF_K + S::KV_TILE);
      const uint64_t v_desc0 = umma_desc_mn_sw128(smem_base + S::OFF_V, A_BKV * 128, 1024);
      const uint64_t v_desc1 = umma_desc_mn_sw128(smem_base + S::OFF_V + S::KV_TILE, A_BKV * 128, 1024);
      static_assert(A_KV_STAGES == 2 && A_BQ == A_BKV, "descriptor selection below assumes two stages");
      auto issue_s = [&](int t, int vb) {
        const uint64_t qd = t ? q_desc1 : q_desc0;
        const uint64_t kd = (vb & 1) ? k_desc1 : k_desc0;
        const uint32_t ds = tm_s[t];
#pragma unroll
        for (int kk = 0; kk < HDP / 16; ++kk) {
          if (kk < k_steps) {
            // 64-column blocks of the head are A_BQ * 128 bytes apart, 16 columns are 32 bytes
            const uint64_t off = static_cast<uint64_t>(((kk >> 2) * (A_BQ * 128) + (kk & 3) * 32) >> 4);
            umma_bf16_ss(ds, qd + off, kd + off, idesc_s, kk != 0);
          }
        }
        umma_commit(smem_u32(&bar_s[t]));
      };
      auto issue_pv = [&](int t, int vb) {
        // A = P from TMEM: 16 keys = 8 packed 32-bit columns.  B = V, MN-major: 16 keys = two
        // 8-row groups of 1024 bytes; 64-column blocks of the head are A_BKV*128 bytes apart.
        const uint64_t vd = (vb & 1) ? v_desc1 : v_desc0;
        const uint32_t dso = tm_o[t], pa = tm_s[t];
#pragma unroll
        for (int kk = 0; kk < A_BKV / 16; ++kk)
          umma_bf16_ts(dso, pa + kk * 8, vd + static_cast<uint64_t>(kk * (2048 >> 4)), idesc_o, (vb | kk) != 0);
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
    // ------------------------------------------------------------ softmax warpgroups
    const int t = warp >> 2;           // query tile of this warpgroup
    const int quad = warp & 3;         // TMEM lane quadrant
    const int r = quad * 32 + lane;    // row inside the tile
    const int qi = q0[t] + r;          // query index inside the sequence
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;

    for (int vb = 0; vb < nvb[t] && ok; ++vb) {
      ok = mbar_wait(smem_u32(&bar_s[t]), vb & 1, &s_abort, p.err, ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const bool is_prefix = has_prefix && vb == 0;
      const int kv0 = (jb + vb - has_prefix) * A_BKV;
      // blocks entirely below the diagonal and right of the padding need no mask (uniform)
      const bool need_mask = is_prefix || !(kv0 + A_BKV - 1 <= q0[t] && kv0 >= pad);
      auto visible = [&](int c) -> bool {
        if (is_prefix) return c < p.n_prefix;
        int kv = kv0 + c;
        return (kv <= qi) && (kv >= pad || kv == qi) && (kv < p.L);
      };
      // ---- the whole score row of this block in registers: one TMEM round trip
      uint32_t sv[A_BKV];
#pragma unroll
      for (int ch = 0; ch < A_BKV / 32; ++ch) tmem_ld_32x32(tm_s[t] + lane_off + ch * 32, sv + ch * 32);
      tmem_ld_wait();
      // four independent chains: a single running maximum would serialise 128 dependent operations
      float bm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < A_BKV; ++c) {
          if (!visible(c)) sv[c] = 0xff800000u;  // -inf
          bm[c & 3] = fmaxf(bm[c & 3], __uint_as_float(sv[c]));
        }
      } else {
#pragma unroll
        for (int c = 0; c < A_BKV; ++c) bm[c & 3] = fmaxf(bm[c & 3], __uint_as_float(sv[c]));
      }
      float bmax = fmaxf(fmaxf(bm[0], bm[1]), fmaxf(bm[2], bm[3]));
      bmax *= p.scale_log2;       // scale > 0: max commutes with the scaling
      // lazily raised maximum
      float m_new = m_used;
      if (bmax > m_used + A_RESCALE_THRESHOLD || m_used == -INFINITY) m_new = fmaxf(m_used, bmax);
      const bool changed = (m_new != m_used);
      if (vb > 0) {
        // PV of the previous block is complete here - O may be touched and P overwritten: it was issued before
        // this block's score product by the same thread, and the commit that signalled bar_s covers every
        // tensor-core operation issued before it
        if (__any_sync(0xffffffffu, changed && m_used != -INFINITY)) {
          const float f = (changed && m_used != -INFINITY) ? exp2f(m_used - m_new) : 1.0f;
          for (int c0 = 0; c0 < hd; c0 += 16) {
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
      // ---- probabilities -> bf16 pairs (packed in place) -> TMEM, over the columns S occupied
      const float mref = (m_used == -INFINITY) ? 0.f : m_used;
      float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < A_BKV; c += 2) {
        float e0 = exp2f(fmaf(__uint_as_float(sv[c]), p.scale_log2, -mref));
        float e1 = exp2f(fmaf(__uint_as_float(sv[c + 1]), p.scale_log2, -mref));
        ps[(c >> 1) & 3] += e0 + e1;
        sv[c >> 1] = pack_bf16x2(e0, e1);
      }
      const float psum = (ps[0] + ps[1]) + (ps[2] + ps[3]);
#pragma unroll
      for (int ch = 0; ch < A_BKV / 32; ++ch) tmem_st_32x16(tm_s[t] + lane_off + ch * 16, sv + ch * 16);
      l_sum += psum;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_p[t]));
    }
    // ---- epilogue: O / l -> bf16 -> global
    if (ok && nvb[t] > 0) {
      ok = mbar_wait(smem_u32(&bar_pv[t]), (nvb[t] - 1) & 1, &s_abort, p.err, ERR_WAIT_MISC);
      if (ok) {
        tc_fence_after();
        const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
        const bool row_ok = qi < p.L;
        if (p.lse && row_ok)
          p.lse[((long long)b * p.H + h) * p.L + qi] = l_sum > 0.f ? m_used + log2f(l_sum) : 0.f;
        __nv_bfloat16* orow = p.out + ((long long)b * p.L + qi) * p.ld_out + h * hd;
        // all accumulator columns in one TMEM round trip (hd is a multiple of 16, <= 128)
        uint32_t o[128];
#pragma unroll
        for (int c0 = 0; c0 < 128; c0 += 16)
          if (c0 < hd) tmem_ld_32x16(tm_o[t] + lane_off + c0, o + c0);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int c0 = 0; c0 < 128; c0 += 8) {
            if (c0 < hd) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(o[c0 + 0]) * inv, __uint_as_float(o[c0 + 1]) * inv);
              w.y = pack_bf16x2(__uint_as_float(o[c0 + 2]) * inv, __uint_as_float(o[c0 + 3]) * inv);
              w.z = pack_bf16x2(__uint_as_float(o[c0 + 4]) * inv, __uint_as_float(o[c0 + 5]) * inv);
              w.w = pack_bf16x2(__uint_as_float(o[c0 + 6]) * inv, __uint_as_float(o[c0 + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c0) = w;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    if (s_abort) {
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int HDP>
static int launch_attn(const CUtensorMap& tmQ, const CUtensorMap& tmKV, const CUtensorMap& tmPK,
                       const CUtensorMap& tmPV, const AttnArgs& a, cudaStream_t stream) {
  using S = AttnSmem<HDP>;
  auto kern = attn_fwd_kernel<HDP>;
  static PerDeviceFlag configured;
  if (int rc_cfg = ensure_dyn_smem(configured, kern, S::TOTAL)) return rc_cfg;
  int pairs = (a.L + 2 * A_BQ - 1) / (2 * A_BQ);
  dim3 grid(pairs, a.H, a.B);
  kern<<<grid, A_THREADS, S::TOTAL, stream>>>(tmQ, tmKV, tmPK, tmPV, a);
  return cuda_rc(cudaGetLastError());
}

}  // namespace dz

using namespace dz;

// qkv: [B*L, ld_qkv] bf16 with Q at columns [q_col0, q_col0 + H*hd), K at k_col0, V at v_col0.
// out: [B*L, ld_out] bf16.  prefix_k / prefix_v: [n_prefix, ld_prefix] bf16 or null.
// hd in {64, 80, 96, 112, 128} (multiple of 16, at most 128); at most 128 prefix rows.
// lse: optional [B, H, L] fp32 output, m + log2(sum) of every query row in the log2 domain of the
// scaled scores (what dz_attn_bwd reads).
extern "C" int dz_attn_fwd_lse(const void* qkv, long long ld_qkv, int q_col0, int k_col0, int v_col0,
                               void* out, long long ld_out, const int* pad_left, const void* prefix_k,
                               const void* prefix_v, long long ld_prefix, int n_prefix, int B, int L,
                               int H, int hd, float scale, float* lse, uint32_t* err, cudaStream_t stream) {
  if (!qkv || !out || B <= 0 || L <= 0 || H <= 0) return DZ_ERR_ARG;
  if (hd < 16 || hd > 128 || (hd & 15)) return DZ_ERR_ARG;
  if (n_prefix < 0 || n_prefix > A_BKV || (n_prefix > 0 && (!prefix_k || !prefix_v)))
    return DZ_ERR_ARG;
  if ((q_col0 | k_col0 | v_col0) & 7) return DZ_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (ld_out & 7)) return DZ_ERR_ALIGN;
  const int hdp = hd <= 64 ? 64 : 128;
  const long long rows = (long long)B * L;
  // logical width of a row as far as any section reaches; TMA zero-fills beyond it
  long long width = ld_qkv;
  CUtensorMap tmQ, tmKV, tmPK, tmPV;
  int rc = make_tmap_bf16_2d(&tmQ, qkv, rows, width, ld_qkv, A_BQ, 64, true);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tmKV, qkv, rows, width, ld_qkv, A_BKV, 64, true);
  if (rc) return rc;
  if (n_prefix > 0) {
    rc = make_tmap_bf16_2d(&tmPK, prefix_k, n_prefix, (long long)H * hd, ld_prefix, A_BKV, 64, true);
    if (rc) return rc;
    rc = make_tmap_bf16_2d(&tmPV, prefix_v, n_prefix, (long long)H * hd, ld_prefix, A_BKV, 64, true);
    if (rc) return rc;
  } else {
    tmPK = tmKV;
    tmPV = tmKV;
  }
  AttnArgs a{};
  a.B = B; a.L = L; a.H = H; a.hd = hd; a.n_prefix = n_prefix; a.ld_out = ld_out;
  a.out = (__nv_bfloat16*)out; a.pad_left = pad_left; a.lse = lse;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.q_col0 = q_col0; a.k_col0 = k_col0; a.v_col0 = v_col0; a.err = err;
  if (hdp == 64) return launch_attn<64>(tmQ, tmKV, tmPK, tmPV, a, stream);
  return launch_attn<128>(tmQ, tmKV, tmPK, tmPV, a, stream);
}

extern "C" int dz_attn_fwd(const void* qkv, long long ld_qkv, int q_col0, int k_col0, int v_col0,
                           void* out, long long ld_out, const int* pad_left, const void* prefix_k,
                           const void* prefix_v, long long ld_prefix, int n_prefix, int B, int L,
                           int H, int hd, float scale, uint32_t* err, cudaStream_t stream) {
  return dz_attn_fwd_lse(qkv, ld_qkv, q_col0, k_col0, v_col0, out, ld_out, pad_left, prefix_k, prefix_v,
                         ld_prefix, n_prefix, B, L, H, hd, scale, nullptr, err, stream);
}
