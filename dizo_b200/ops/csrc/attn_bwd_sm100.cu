// Backward of the causal self-attention of attn_sm100.cu for sm_100a (tcgen05 + TMEM).
//
// Given Q, K, V (in place inside the fused QKV activation), the context O, its gradient dO and
// the per-row log-sum-exp the forward saved, produces dQ, dK and dV in the layout of the QKV
// activation, so the gradient GEMM of the fused QKV projection consumes them directly.  Used by
// the first-order gamma search of DiZO (large_models/trainer.py:714-741, :805-830), which needs
// d loss / d (k_proj, v_proj weights) and therefore the gradient through every attention block.
// The reference obtains these from autograd over the bmm / softmax / bmm chain of
// large_models/ht_opt.py:209-272.
//
// Two passes of one templated kernel, both without atomics (deterministic):
//   DQ = false : one CTA owns a 128-key tile (K_j, V_j stationary in shared memory) and streams
//                the query tiles i >= j:   S^T = K_j Q_i^T,  dP^T = V_j dO_i^T   (both in TMEM)
//                P^T = exp2(S^T * c - lse_i),  dS^T = P^T * (dP^T - D_i)   (bf16, back into TMEM)
//                dV_j += P^T dO_i,  dK_j += dS^T Q_i      (P^T / dS^T as the TMEM A operand)
//   DQ = true  : one CTA owns a 128-query tile (Q_i, dO_i stationary) and streams the key tiles
//                j <= i:   S = Q_i K_j^T,  dP = dO_i V_j^T,  dS = P * (dP - D_i),  dQ_i += dS K_j
// D = rowsum(dO * O) comes from a small preparation kernel.  The 1/sqrt(hd) scale is applied in
// the epilogue (dQ, dK).  Masking is the forward's: key j visible to query i iff j <= i and
// (j >= pad_left or j == i).
//
// Warps 0-7: softmax arithmetic and epilogue - a thread owns one stationary row and one 64-column
// half of the streamed tile (warps w and w+4 share a TMEM lane quadrant and split the columns);
// warp 8: TMEM allocation, lane 0 issues tcgen05.mma; warp 9: lane 0 is the TMA producer.
#include "common.cuh"
#include "host_util.h"

namespace dz {

constexpr int AB_T = 128;          // rows of a stationary or streamed tile
constexpr int AB_THREADS = 320;
constexpr int AB_STAGES = 2;

struct AttnBwdArgs {
  int B, L, H, hd;
  const int* pad_left;
  const float* lse;          // [B, H, L], log2 domain: m + log2(sum)
  const float* dsum;         // [B, H, L], rowsum(dO * O)
  __nv_bfloat16* dqkv;       // [B*L, ld_dqkv]
  long long ld_dqkv;
  int q_col0, k_col0, v_col0;
  float scale, scale_log2;
  uint32_t* err;
};

template <int HDP>
struct AttnBwdSmem {
  static constexpr int TILE = AB_T * HDP * 2;
  static constexpr int OFF_X1 = 0;
  static constexpr int OFF_X2 = TILE;
  static constexpr int OFF_Y1 = 2 * TILE;                       // AB_STAGES stages
  static constexpr int OFF_Y2 = OFF_Y1 + AB_STAGES * TILE;
  static constexpr int USED = OFF_Y2 + AB_STAGES * TILE + 1024;
  // at least 120 KB so that two CTAs (each wanting all 512 TMEM columns) never share an SM
  static constexpr int TOTAL = USED < 120 * 1024 ? 120 * 1024 : USED;
};

template <int HDP, bool DQ>
__global__ void __launch_bounds__(AB_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO,
                const AttnBwdArgs p) {
  using S = AttnBwdSmem<HDP>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_x;
  __shared__ __align__(8) uint64_t bar_y_full[AB_STAGES], bar_y_empty[AB_STAGES];
  __shared__ __align__(8) uint64_t bar_s, bar_ds, bar_acc;
  __shared__ float4 s_stat[8][32];      // per softmax warp: {lse, D, lse, D} of its 64 streamed rows, two per entry
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile int s_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int nT = (p.L + AB_T - 1) / AB_T;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int pad = p.pad_left ? p.pad_left[b] : 0;
  const int hd = p.hd;
  // stationary tile (heaviest first) and the range of streamed tiles [y_lo, y_hi)
  const int xt = DQ ? nT - 1 - (int)blockIdx.x : (int)blockIdx.x;
  const int x0 = xt * AB_T;
  const int y_lo = DQ ? min(pad, x0) / AB_T : xt;
  const int y_hi = DQ ? xt + 1 : nT;
  const int n_it = y_hi - y_lo;
  const int row_base = b * p.L;
  // columns of the stationary / streamed operands inside the QKV rows
  const int x1_col = (DQ ? p.q_col0 : p.k_col0) + h * hd;   // Q_i | K_j
  const int y1_col = (DQ ? p.k_col0 : p.q_col0) + h * hd;   // K_j | Q_i
  const int v_col = p.v_col0 + h * hd;
  const int do_col = h * hd;

  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(smem_u32(&bar_x), 1);
    for (int s = 0; s < AB_STAGES; ++s) {
      mbar_init(smem_u32(&bar_y_full[s]), 1);
      mbar_init(smem_u32(&bar_y_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_s), 1);
    mbar_init(smem_u32(&bar_ds), 8);
    mbar_init(smem_u32(&bar_acc), 1);
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
  // TMEM columns: S / P [0,128), dP / dS [128,256), accumulator 1 [256,256+HDP), accumulator 2 [384,..)
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128u;
  const uint32_t tm_acc1 = tmem_base + 256u, tm_acc2 = tmem_base + 384u;

  if (warp == 9) {
    if (lane == 0 && n_it > 0) {
      // ---------------------------------------------- TMA producer
      // stationary: X1 = Q_i | K_j,  X2 = dO_i | V_j
      mbar_arrive_expect_tx(smem_u32(&bar_x), 2 * S::TILE);
      for (int c = 0; c < HDP / 64; ++c) {
        tma_load_2d(smem_base + S::OFF_X1 + c * (AB_T * 128), &tmQKV, smem_u32(&bar_x), x1_col + c * 64,
                    row_base + x0);
        if (DQ)
          tma_load_2d(smem_base + S::OFF_X2 + c * (AB_T * 128), &tmDO, smem_u32(&bar_x), do_col + c * 64,
                      row_base + x0);
        else
          tma_load_2d(smem_base + S::OFF_X2 + c * (AB_T * 128), &tmQKV, smem_u32(&bar_x), v_col + c * 64,
                      row_base + x0);
      }
      // streamed: Y1 = K_j | Q_i,  Y2 = V_j | dO_i
      for (int it = 0; it < n_it; ++it) {
        const int st = it % AB_STAGES;
        const uint32_t ph = (it / AB_STAGES) & 1;
        const int yrow = row_base + (y_lo + it) * AB_T;
        if (!mbar_wait(smem_u32(&bar_y_empty[st]), ph ^ 1, &s_abort, p.err, ERR_WAIT_EMPTY)) break;
        uint32_t full = smem_u32(&bar_y_full[st]);
        mbar_arrive_expect_tx(full, 2 * S::TILE);
        for (int c = 0; c < HDP / 64; ++c) {
          tma_load_2d(smem_base + S::OFF_Y1 + st * S::TILE + c * (AB_T * 128), &tmQKV, full, y1_col + c * 64,
                      yrow);
          if (DQ)
            tma_load_2d(smem_base + S::OFF_Y2 + st * S::TILE + c * (AB_T * 128), &tmQKV, full, v_col + c * 64,
                        yrow);
          else
            tma_load_2d(smem_base + S::OFF_Y2 + st * S::TILE + c * (AB_T * 128), &tmDO, full, do_col + c * 64,
                        yrow);
        }
      }
    }
  } else if (warp == 8) {
    if (lane == 0 && n_it > 0) {
      // ---------------------------------------------- MMA issuer
      const uint32_t idesc_s = umma_idesc_bf16(AB_T, AB_T, 0, 0);
      const uint32_t idesc_acc = umma_idesc_bf16(AB_T, (hd + 15) & ~15, 0, 1);   // B operand MN-major
      const int k_steps = (hd + 15) / 16;
      bool ok = mbar_wait(smem_u32(&bar_x), 0, &s_abort, p.err, ERR_WAIT_FULL);
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it % AB_STAGES;
        const uint32_t ph = (it / AB_STAGES) & 1;
        ok = mbar_wait(smem_u32(&bar_y_full[st]), ph, &s_abort, p.err, ERR_WAIT_FULL);
        if (!ok) break;
        tc_fence_after();
        // One thread issues every MMA and a 128 x 128 x 16 product lasts 64 cycles, so the descriptors are
        // built once per iteration and each MMA only adds a constant to their address field.
        const uint64_t x1d = umma_desc_k_sw128(smem_base + S::OFF_X1), x2d = umma_desc_k_sw128(smem_base + S::OFF_X2);
        const uint32_t y1 = smem_base + S::OFF_Y1 + st * S::TILE, y2 = smem_base + S::OFF_Y2 + st * S::TILE;
        const uint64_t y1d = umma_desc_k_sw128(y1), y2d = umma_desc_k_sw128(y2);
        const uint64_t y1m = umma_desc_mn_sw128(y1, AB_T * 128, 1024), y2m = umma_desc_mn_sw128(y2, AB_T * 128, 1024);
        // S (or S^T) = X1 Y1^T,  dP (or dP^T) = X2 Y2^T : contraction over the head dimension.
        // Tensor-core operations of one thread execute in issue order, so these overwrite the
        // S / dP columns only after the previous iteration's accumulations have read them.
#pragma unroll
        for (int kk = 0; kk < HDP / 16; ++kk) {
          if (kk < k_steps) {
            const uint64_t off = static_cast<uint64_t>(((kk >> 2) * (AB_T * 128) + (kk & 3) * 32) >> 4);
            umma_bf16_ss(tm_s, x1d + off, y1d + off, idesc_s, kk != 0);
          }
        }
#pragma unroll
        for (int kk = 0; kk < HDP / 16; ++kk) {
          if (kk < k_steps) {
            const uint64_t off = static_cast<uint64_t>(((kk >> 2) * (AB_T * 128) + (kk & 3) * 32) >> 4);
            umma_bf16_ss(tm_dp, x2d + off, y2d + off, idesc_s, kk != 0);
          }
        }
        umma_commit(smem_u32(&bar_s));
        ok = mbar_wait(smem_u32(&bar_ds), it & 1, &s_abort, p.err, ERR_WAIT_MISC);
        if (!ok) break;
        tc_fence_after();
        // contraction over the 128 streamed rows: 16 rows = 8 packed TMEM columns of the A operand
        // (rows 0-63 packed at columns [0,32), rows 64-127 at [64,96)) and two 8-row groups
        // (1024 bytes each) of the MN-major B operand
        if (!DQ) {
#pragma unroll
          for (int kk = 0; kk < AB_T / 16; ++kk)      // dV_j += P^T dO_i
            umma_bf16_ts(tm_acc1, tm_s + (kk >> 2) * 64 + (kk & 3) * 8, y2m + static_cast<uint64_t>(kk * (2048 >> 4)),
                         idesc_acc, (it | kk) != 0);
        }
#pragma unroll
        for (int kk = 0; kk < AB_T / 16; ++kk)        // dK_j += dS^T Q_i   |   dQ_i += dS K_j
          umma_bf16_ts(DQ ? tm_acc1 : tm_acc2, tm_dp + (kk >> 2) * 64 + (kk & 3) * 8,
                       y1m + static_cast<uint64_t>(kk * (2048 >> 4)), idesc_acc, (it | kk) != 0);
        umma_commit(smem_u32(&bar_y_empty[st]));
      }
      if (ok) umma_commit(smem_u32(&bar_acc));
    }
  } else {
    // ---------------------------------------------- softmax arithmetic: one stationary row, 64 columns
    const int quad = warp & 3;                              // TMEM lane quadrant
    const int half = warp >> 2;                             // which 64 streamed rows (columns of S)
    const int r = quad * 32 + lane;
    const int xi = x0 + r;                                  // key index (DQ false) | query index (DQ true)
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const long long stat_base = ((long long)b * p.H + h) * p.L;
    float my_lse = 0.f, my_dsum = 0.f;
    if (DQ && xi < p.L) {
      my_lse = p.lse[stat_base + xi];
      my_dsum = p.dsum[stat_base + xi];
    }
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int y0 = (y_lo + it) * AB_T;
      if (!DQ) {
        // statistics of the streamed query rows, one private copy per warp (the __syncwarp that
        // ends every iteration orders these writes after the previous iteration's reads)
        {
          const int q0 = y0 + half * 64 + lane * 2;
          float4 st;
          st.x = q0 < p.L ? p.lse[stat_base + q0] : 0.f;
          st.y = q0 < p.L ? p.dsum[stat_base + q0] : 0.f;
          st.z = q0 + 1 < p.L ? p.lse[stat_base + q0 + 1] : 0.f;
          st.w = q0 + 1 < p.L ? p.dsum[stat_base + q0 + 1] : 0.f;
          s_stat[warp][lane] = st;
        }
        __syncwarp();
      }
      ok = mbar_wait(smem_u32(&bar_s), it & 1, &s_abort, p.err, ERR_WAIT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);          // leave the loop as a whole warp
      if (!ok) break;
      tc_fence_after();
      {
        uint32_t sv[64], dv[64];
        tmem_ld_32x32(tm_s + lane_off + half * 64, sv);
        tmem_ld_32x32(tm_s + lane_off + half * 64 + 32, sv + 32);
        tmem_ld_32x32(tm_dp + lane_off + half * 64, dv);
        tmem_ld_32x32(tm_dp + lane_off + half * 64 + 32, dv + 32);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          float pr[2], dsv[2];
          float4 st = make_float4(0.f, 0.f, 0.f, 0.f);
          if (!DQ) st = s_stat[warp][c >> 1];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int yi = y0 + half * 64 + c + u;
            const int kv = DQ ? yi : xi;
            const int qi = DQ ? xi : yi;
            const bool vis = (kv <= qi) && (kv >= pad || kv == qi) && (qi < p.L);
            const float l = DQ ? my_lse : (u ? st.z : st.x);
            const float dd = DQ ? my_dsum : (u ? st.w : st.y);
            const float pe = vis ? exp2f(fmaf(__uint_as_float(sv[c + u]), p.scale_log2, -l)) : 0.f;
            pr[u] = pe;
            dsv[u] = pe * (__uint_as_float(dv[c + u]) - dd);
          }
          sv[c >> 1] = pack_bf16x2(pr[0], pr[1]);
          dv[c >> 1] = pack_bf16x2(dsv[0], dsv[1]);
        }
        // packed results go back over the first 32 of the 64 columns this warp has just read (never
        // over columns that the other warp of the quadrant reads)
        if (!DQ) {
          tmem_st_32x16(tm_s + lane_off + half * 64, sv);
          tmem_st_32x16(tm_s + lane_off + half * 64 + 16, sv + 16);
        }
        tmem_st_32x16(tm_dp + lane_off + half * 64, dv);
        tmem_st_32x16(tm_dp + lane_off + half * 64 + 16, dv + 16);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_ds));
    }
    // ---- epilogue: accumulators -> bf16 -> the QKV-shaped gradient
    if (ok && n_it > 0) {
      ok = mbar_wait(smem_u32(&bar_acc), 0, &s_abort, p.err, ERR_WAIT_MISC);
      if (ok) {
        tc_fence_after();
        const bool row_ok = xi < p.L;
        __nv_bfloat16* grow = p.dqkv + ((long long)row_base + xi) * p.ld_dqkv;
        for (int which = 0; which < (DQ ? 1 : 2); ++which) {
          // DQ: dQ (scaled).  Otherwise accumulator 1 = dV, accumulator 2 = dK (scaled).
          const uint32_t tm = which == 0 ? tm_acc1 : tm_acc2;
          const float f = (DQ || which == 1) ? p.scale : 1.0f;
          const int col0 = (DQ ? p.q_col0 : (which == 0 ? p.v_col0 : p.k_col0)) + h * hd;
          for (int c0 = half * 16; c0 < hd; c0 += 32) {       // the two warps of a quadrant alternate
            uint32_t o[16];
            tmem_ld_32x16(tm + lane_off + c0, o);
            tmem_ld_wait();
            if (row_ok) {
              uint4 w0, w1;
              w0.x = pack_bf16x2(__uint_as_float(o[0]) * f, __uint_as_float(o[1]) * f);
              w0.y = pack_bf16x2(__uint_as_float(o[2]) * f, __uint_as_float(o[3]) * f);
              w0.z = pack_bf16x2(__uint_as_float(o[4]) * f, __uint_as_float(o[5]) * f);
              w0.w = pack_bf16x2(__uint_as_float(o[6]) * f, __uint_as_float(o[7]) * f);
              w1.x = pack_bf16x2(__uint_as_float(o[8]) * f, __uint_as_float(o[9]) * f);
              w1.y = pack_bf16x2(__uint_as_float(o[10]) * f, __uint_as_float(o[11]) * f);
              w1.z = pack_bf16x2(__uint_as_float(o[12]) * f, __uint_as_float(o[13]) * f);
              w1.w = pack_bf16x2(__uint_as_float(o[14]) * f, __uint_as_float(o[15]) * f);
              *reinterpret_cast<uint4*>(grow + col0 + c0) = w0;
              *reinterpret_cast<uint4*>(grow + col0 + c0 + 8) = w1;
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

// D[b, h, l] = sum_c dO[b, l, h*hd + c] * O[b, l, h*hd + c]; one warp per (row, head).
__global__ void attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                     long long ld, float* __restrict__ dsum, int B, int L, int H, int hd) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)B * L * H) return;
  const int hh = (int)(w % H);
  const long long row = w / H;
  const __nv_bfloat16* po = o + row * ld + hh * hd;
  const __nv_bfloat16* pd = d_o + row * ld + hh * hd;
  float acc = 0.f;
  for (int c = lane * 2; c < hd; c += 64) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(po + c);
    const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(pd + c);
    acc = fmaf(__bfloat162float(a.x), __bfloat162float(g.x), acc);
    acc = fmaf(__bfloat162float(a.y), __bfloat162float(g.y), acc);
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) {
    const long long bb = row / L, l = row % L;
    dsum[(bb * H + hh) * L + l] = acc;
  }
}

template <int HDP, bool DQ>
static int launch_attn_bwd(const CUtensorMap& tmQKV, const CUtensorMap& tmDO, const AttnBwdArgs& a,
                           cudaStream_t stream) {
  using S = AttnBwdSmem<HDP>;
  auto kern = attn_bwd_kernel<HDP, DQ>;
  static PerDeviceFlag configured;
  if (int rc_cfg = ensure_dyn_smem(configured, kern, S::TOTAL)) return rc_cfg;
  dim3 grid((a.L + AB_T - 1) / AB_T, a.H, a.B);
  kern<<<grid, AB_THREADS, S::TOTAL, stream>>>(tmQKV, tmDO, a);
  return cuda_rc(cudaGetLastError());
}

}  // namespace dz

using namespace dz;

// qkv [B*L, ld_qkv] bf16 as in dz_attn_fwd (no prefix rows); out / dout [B*L, ld_out] bf16: the
// forward's context and its gradient; lse [B, H, L] fp32 from dz_attn_fwd_lse; dsum [B, H, L]
// fp32 scratch (written here); dqkv [B*L, ld_dqkv] bf16 receives dQ, dK, dV at q_col0 / k_col0 /
// v_col0.  hd a multiple of 16, at most 128.
extern "C" int dz_attn_bwd(const void* qkv, long long ld_qkv, int q_col0, int k_col0, int v_col0,
                           const void* out, const void* dout, long long ld_out, const float* lse,
                           float* dsum, void* dqkv, long long ld_dqkv, const int* pad_left, int B, int L,
                           int H, int hd, float scale, uint32_t* err, cudaStream_t stream) {
  if (!qkv || !out || !dout || !lse || !dsum || !dqkv || B <= 0 || L <= 0 || H <= 0) return DZ_ERR_ARG;
  if (hd < 16 || hd > 128 || (hd & 15)) return DZ_ERR_ARG;
  if ((q_col0 | k_col0 | v_col0) & 7) return DZ_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(dqkv) & 15) || (ld_dqkv & 7) || (ld_out & 7)) return DZ_ERR_ALIGN;
  const long long rows = (long long)B * L;
  {
    const long long warps = rows * H;
    const int threads = 256;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    attn_bwd_prep_kernel<<<(unsigned)blocks, threads, 0, stream>>>(
        (const __nv_bfloat16*)out, (const __nv_bfloat16*)dout, ld_out, dsum, B, L, H, hd);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_rc(e);
  }
  CUtensorMap tmQKV, tmDO;
  int rc = make_tmap_bf16_2d(&tmQKV, qkv, rows, ld_qkv, ld_qkv, AB_T, 64, true);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tmDO, dout, rows, ld_out, ld_out, AB_T, 64, true);
  if (rc) return rc;
  AttnBwdArgs a{};
  a.B = B; a.L = L; a.H = H; a.hd = hd; a.pad_left = pad_left; a.lse = lse; a.dsum = dsum;
  a.dqkv = (__nv_bfloat16*)dqkv; a.ld_dqkv = ld_dqkv;
  a.q_col0 = q_col0; a.k_col0 = k_col0; a.v_col0 = v_col0;
  a.scale = scale; a.scale_log2 = scale * 1.4426950408889634f; a.err = err;
  const int hdp = hd <= 64 ? 64 : 128;
  if (hdp == 64) {
    rc = launch_attn_bwd<64, false>(tmQKV, tmDO, a, stream);
    if (rc) return rc;
    return launch_attn_bwd<64, true>(tmQKV, tmDO, a, stream);
  }
  rc = launch_attn_bwd<128, false>(tmQKV, tmDO, a, stream);
  if (rc) return rc;
  return launch_attn_bwd<128, true>(tmQKV, tmDO, a, stream);
}
