// Two-SM variant of the bf16 GEMM:  out[M,N] = epilogue( A[M,K] * W[N,K]^T ).
//
// A thread-block cluster of two CTAs (one per SM of a pair) computes one 256 x 256 output
// tile with tcgen05.mma.cta_group::2: CTA r of the pair stages rows [128r, 128r+128) of the
// A tile and rows [128r, 128r+128) of the W tile, so each SM fills 32 KB per 64-wide K block
// instead of the 48 KB of the one-SM kernel (gemm_sm100.cu) while the pair issues
// 256 x 256 x 16 instructions that read both halves from both shared memories.  The
// accumulator of CTA r (its 128 rows x 256 columns, fp32) lives in that CTA's TMEM, double
// buffered, and is drained by that CTA's own epilogue warps.
//
//   warp 0   : TMA producer of this CTA (loads carry .cta_group::2 and complete on the
//              LEADER's "full" barrier; no multicast anywhere)
//   warp 1   : TMEM allocation (both CTAs); in the leader, one lane issues the MMAs and
//              commits to the ring's "empty" barriers and the accumulator "full" barriers of
//              BOTH CTAs (tcgen05.commit ... multicast::cluster)
//   warps 2-5: epilogue of this CTA's 128 rows; hands the accumulator back by arriving on
//              the leader's "accumulator empty" barrier (count 8 = 4 warps x 2 CTAs)
// Every wait is bounded (see common.cuh); both CTAs meet at a cluster barrier before TMEM is
// released, so neither exits while the other may still read its shared memory.
#include <stdlib.h>
#include "common.cuh"
#include "cluster2sm.cuh"
#include "host_util.h"

namespace dz {

constexpr int G2_BM = 256;   // per cluster
constexpr int G2_BN = 256;
constexpr int G2_BK = 64;
constexpr int G2_STAGES = 6;
constexpr int G2_THREADS = 192;
constexpr int G2_A_BYTES = 128 * G2_BK * 2;          // this CTA's half of A
constexpr int G2_B_BYTES = (G2_BN / 2) * G2_BK * 2;  // this CTA's half of W
constexpr int G2_STAGE_BYTES = G2_A_BYTES + G2_B_BYTES;
constexpr int G2_SMEM = G2_STAGES * G2_STAGE_BYTES + 1024;
constexpr uint32_t G2_TMEM_COLS = 2 * G2_BN;

struct Gemm2Args {
  int M, N, K;
  int num_m, num_n, group_m;
  void* out;
  long long ldo;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  long long ldr;
  int act;
  int out_fp32;
  float out_scale;
  uint32_t* err;
  // act 4: rotary embedding of a fused q | k | v projection in the epilogue (head dim 128)
  int wide_store;           // out and its row pitch are 32-byte aligned: 256-bit stores in the bf16 epilogues
  int wide_residual;        // the same for the residual rows: 256-bit loads
  const float* rope_cs;     // fp32 [n_pos][64][2] = (cos, sin)
  int rope_L, rope_pos0, rope_n_pos, rope_H, rope_Hkv;
};

__device__ __forceinline__ void tile_coords2(int tile, const Gemm2Args& p, int& mb, int& nb) {
  int tiles_per_group = p.group_m * p.num_n;
  int g = tile / tiles_per_group;
  int first_m = g * p.group_m;
  int gm = min(p.group_m, p.num_m - first_m);
  int r = tile - g * tiles_per_group;
  mb = first_m + r % gm;
  nb = r / gm;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G2_THREADS, 1)
gemm2_bf16_tn_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const Gemm2Args p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[G2_STAGES];    // used in the leader only
  __shared__ __align__(8) uint64_t bar_empty[G2_STAGES];   // one per CTA
  __shared__ __align__(8) uint64_t bar_acc_full[2];        // one per CTA
  __shared__ __align__(8) uint64_t bar_acc_empty[2];       // used in the leader only
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile int s_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int num_tiles = p.num_m * p.num_n;
  const int num_kb = (p.K + G2_BK - 1) / G2_BK;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < G2_STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_acc_full[a]), 1);
      mbar_init(smem_u32(&bar_acc_empty[a]), 8);
    }
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_2sm(smem_u32(&s_tmem_base), G2_TMEM_COLS);
    tmem_relinquish_2sm();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // peer barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (each CTA)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        int mb, nb;
        tile_coords2(tile, p, mb, nb);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1, &s_abort, p.err, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t full_local = smem_u32(&bar_full[stage]);
          const uint32_t full_leader = map_to_cta(full_local, 0);
          const uint32_t a_dst = smem_base + stage * G2_STAGE_BYTES;
          const uint32_t b_dst = a_dst + G2_A_BYTES;
          if (leader) mbar_arrive_expect_tx(full_local, 2 * G2_STAGE_BYTES);  // both CTAs' bytes
          tma_load_2d_2sm(a_dst, &tmA, full_leader, kb * G2_BK, mb * G2_BM + (int)rank * 128);
          // act 3 (SwiGLU over W = gate rows | up rows): the leader's half of the tile is 128 gate rows, the
          // peer's half the matching 128 up rows, so that column j and column 128 + j of the accumulator pair up
          const int b_row = p.act == 3 ? (int)rank * (p.N >> 1) + nb * (G2_BN / 2)
                                       : nb * G2_BN + (int)rank * (G2_BN / 2);
          tma_load_2d_2sm(b_dst, &tmB, full_leader, kb * G2_BK, b_row);
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA)
    if (leader && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(G2_BM, G2_BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        if (!mbar_wait_cluster(smem_u32(&bar_acc_empty[acc]), acc_phase ^ 1, &s_abort, p.err,
                               ERR_WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * G2_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &s_abort, p.err, ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_src = smem_base + stage * G2_STAGE_BYTES;
          const uint32_t b_src = a_src + G2_A_BYTES;
          const uint64_t a_desc = umma_desc_k_sw128(a_src);
          const uint64_t b_desc = umma_desc_k_sw128(b_src);
#pragma unroll
          for (int k = 0; k < G2_BK / 16; ++k)
            umma_bf16_ss_2sm(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
          umma_commit_2sm(smem_u32(&bar_empty[stage]), 3);     // frees the stage in both CTAs
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_2sm(smem_u32(&bar_acc_full[acc]), 3);      // wakes both epilogues
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (each CTA)
    const int quad = warp & 3;
    const int row_in_tile = (int)rank * 128 + quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = cluster_id; tile < num_tiles; tile += num_clusters) {
      int mb, nb;
      tile_coords2(tile, p, mb, nb);
      if (!mbar_wait(smem_u32(&bar_acc_full[acc]), acc_phase, &s_abort, p.err, ERR_WAIT_TMEM_FULL))
        break;
      tc_fence_after();
      const long long row = (long long)mb * G2_BM + row_in_tile;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + acc * G2_BN + (static_cast<uint32_t>(quad * 32) << 16);
      if (p.act == 4) {
        // The tile holds two heads of 128 columns of q | k | v (raw layout: H query heads, Hkv key heads, Hkv value
        // heads).  q and k heads are rotated - columns j and j + 64 of a head pair up, angle from the row's position
        // and j - and written to the expanded layout [q: H heads | k: H heads | v: H heads], k / v heads repeated
        // H / Hkv times; v heads are copied.
        const int H = p.rope_H, Hkv = p.rope_Hkv, rep = H / Hkv;
        int pos = p.rope_pos0 + (int)(row % p.rope_L);
        pos = pos < p.rope_n_pos ? pos : p.rope_n_pos - 1;
        const float4* csr = reinterpret_cast<const float4*>(p.rope_cs + (long long)pos * 128);
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.ldo;
        auto store32 = [&](int head_out, int n_rep, int col, const float* v) {
          // 32 consecutive columns of one head, to n_rep consecutive output heads
          uint4 o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            o[q].x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]); o[q].y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
            o[q].z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]); o[q].w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
          }
          for (int r = 0; r < n_rep; ++r)
            store_row32(orow + (long long)(head_out + r) * 128 + col, o, p.wide_store != 0);
        };
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {
          const int g = nb * 2 + hh;                    // head in the raw layout
          const bool is_q = g < H, is_k = !is_q && g < H + Hkv;
          const int head_out = is_q ? g : (is_k ? H + (g - H) * rep : 2 * H + (g - H - Hkv) * rep);
          const int n_rep = is_q ? 1 : rep;
#pragma unroll 1
          for (int pc = 0; pc < 2; ++pc) {
            uint32_t a[32], b[32];
            __syncwarp();                                 // lanes of rows past M skipped the stores above
            tmem_ld_32x32(t_row + hh * 128 + pc * 32, a);
            tmem_ld_32x32(t_row + hh * 128 + 64 + pc * 32, b);
            tmem_ld_wait();
            if (!row_ok) continue;
            float lo[32], hi[32];
            if (is_q || is_k) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float4 c = __ldg(csr + pc * 16 + i);       // (cos, sin) of frequencies 2i and 2i + 1
                const float a0 = __uint_as_float(a[2 * i]), a1 = __uint_as_float(a[2 * i + 1]);
                const float b0 = __uint_as_float(b[2 * i]), b1 = __uint_as_float(b[2 * i + 1]);
                lo[2 * i] = a0 * c.x - b0 * c.y;      lo[2 * i + 1] = a1 * c.z - b1 * c.w;
                hi[2 * i] = b0 * c.x + a0 * c.y;      hi[2 * i + 1] = b1 * c.z + a1 * c.w;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) { lo[i] = __uint_as_float(a[i]); hi[i] = __uint_as_float(b[i]); }
            }
            store32(head_out, n_rep, pc * 32, lo);
            store32(head_out, n_rep, 64 + pc * 32, hi);
          }
        }
      } else if (p.act == 3) {
        // out[row, nb * 128 + j] = silu(gate_j) * up_j from the fp32 accumulators, one rounding to bf16
#pragma unroll 1
        for (int c = 0; c < G2_BN / 64; ++c) {
          uint32_t g[32], u[32];
          __syncwarp();                                   // lanes of rows past M skipped the stores above
          tmem_ld_32x32(t_row + c * 32, g);
          tmem_ld_32x32(t_row + G2_BN / 2 + c * 32, u);
          tmem_ld_wait();
          if (!row_ok) continue;
          auto f = [](uint32_t a, uint32_t b) {
            const float x = __uint_as_float(a);
            return x / (1.f + __expf(-x)) * __uint_as_float(b);
          };
          uint4 o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            o[q].x = pack_bf16x2(f(g[q * 8 + 0], u[q * 8 + 0]), f(g[q * 8 + 1], u[q * 8 + 1]));
            o[q].y = pack_bf16x2(f(g[q * 8 + 2], u[q * 8 + 2]), f(g[q * 8 + 3], u[q * 8 + 3]));
            o[q].z = pack_bf16x2(f(g[q * 8 + 4], u[q * 8 + 4]), f(g[q * 8 + 5], u[q * 8 + 5]));
            o[q].w = pack_bf16x2(f(g[q * 8 + 6], u[q * 8 + 6]), f(g[q * 8 + 7], u[q * 8 + 7]));
          }
          store_row32(reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.ldo + nb * (G2_BN / 2) + c * 32, o,
                      p.wide_store != 0);
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < G2_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = nb * G2_BN + c * 32;
        if (col0 >= p.N) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        const bool full_chunk = (col0 + 32 <= p.N);
        if (p.bias) {
          if (full_chunk) {
            const uint4* bp = reinterpret_cast<const uint4*>(p.bias + col0);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 b = __ldg(bp + q);
              v[q * 8 + 0] += bf16_lo(b.x); v[q * 8 + 1] += bf16_hi(b.x);
              v[q * 8 + 2] += bf16_lo(b.y); v[q * 8 + 3] += bf16_hi(b.y);
              v[q * 8 + 4] += bf16_lo(b.z); v[q * 8 + 5] += bf16_hi(b.z);
              v[q * 8 + 6] += bf16_lo(b.w); v[q * 8 + 7] += bf16_hi(b.w);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
          }
        }
        if (p.out_scale != 1.0f) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= p.out_scale;
        }
        if (p.act == 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
        } else if (p.act == 2) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
        }
        if (row_ok) {
          if (p.residual) {
            const __nv_bfloat16* rp = p.residual + row * p.ldr + col0;
            if (full_chunk && p.wide_residual) {
              // one whole 32-byte sector per lane and load
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                uint32_t b[8];
                asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                             : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]), "=r"(b[6]),
                               "=r"(b[7])
                             : "l"(rp + h * 16));
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  v[h * 16 + 2 * j] += bf16_lo(b[j]);
                  v[h * 16 + 2 * j + 1] += bf16_hi(b[j]);
                }
              }
            } else if (full_chunk) {
              const uint4* rp4 = reinterpret_cast<const uint4*>(rp);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 b = __ldg(rp4 + q);
                v[q * 8 + 0] += bf16_lo(b.x); v[q * 8 + 1] += bf16_hi(b.x);
                v[q * 8 + 2] += bf16_lo(b.y); v[q * 8 + 3] += bf16_hi(b.y);
                v[q * 8 + 4] += bf16_lo(b.z); v[q * 8 + 5] += bf16_hi(b.z);
                v[q * 8 + 6] += bf16_lo(b.w); v[q * 8 + 7] += bf16_hi(b.w);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) v[j] += __bfloat162float(rp[j]);
            }
          }
          if (p.out_fp32) {
            float* op = reinterpret_cast<float*>(p.out) + row * p.ldo + col0;
            if (full_chunk) {
              float4* op4 = reinterpret_cast<float4*>(op);
#pragma unroll
              for (int q = 0; q < 8; ++q)
                if (DZ_STORE_OK(op4 + q, 16)) op4[q] = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N && DZ_STORE_OK(op + j, 4)) op[j] = v[j];
            }
          } else {
            __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.ldo + col0;
            if (full_chunk) {
              uint4 o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                o[q].x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
                o[q].y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
                o[q].z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
                o[q].w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              }
              store_row32(op, o, p.wide_store != 0);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N && DZ_STORE_OK(op + j, 2)) op[j] = __float2bfloat16(v[j]);
            }
          }
        }
      }
      }
      // this CTA's half of the accumulator is drained: tell the leader's MMA issuer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bar_acc_empty[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // ---------------------------------------------------------------- tear-down
  tc_fence_before();
  __syncthreads();
  if (s_abort && threadIdx.x == 0) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, G2_TMEM_COLS);
  }
}

}  // namespace dz

using namespace dz;
DZ_DEBUG_TU(gemm2)

static int gemm2_launch(const void* A, long long lda, const void* W, long long ldw, void* out,
                        long long ldo, const void* bias, const void* residual, long long ldr,
                        int M, int N, int K, int act, int out_fp32, float out_scale,
                        uint32_t* err, cudaStream_t stream, const Gemm2Args* rope);

// Same contract as dz_gemm_bf16_tn (gemm_sm100.cu); computed by pairs of SMs.
extern "C" int dz_gemm2_bf16_tn(const void* A, long long lda, const void* W, long long ldw, void* out,
                                long long ldo, const void* bias, const void* residual, long long ldr,
                                int M, int N, int K, int act, int out_fp32, float out_scale,
                                uint32_t* err, cudaStream_t stream) {
  if (act == 4) return DZ_ERR_ARG;
  return gemm2_launch(A, lda, W, ldw, out, ldo, bias, residual, ldr, M, N, K, act, out_fp32, out_scale, err,
                      stream, nullptr);
}

// Fused q | k | v projection with the rotary embedding in the epilogue: A [M, K], W [(H + 2 Hkv) * 128, K] ->
// out [M, 3 * H * 128] bf16 (q | k | v with the k / v heads repeated H / Hkv times), row m at position
// pos0 + m % L; cs: fp32 [n_pos][64][2] (cos, sin).  Head dim 128, H and Hkv even.
extern "C" int dz_gemm2_qkv_rope(const void* A, long long lda, const void* W, long long ldw, void* out,
                                 long long ldo, const float* cs, int M, int K, int L, int pos0, int n_pos,
                                 int H, int Hkv, uint32_t* err, cudaStream_t stream) {
  if (!cs || L <= 0 || pos0 < 0 || n_pos < pos0 + L || H <= 0 || Hkv <= 0 || (H & 1) || (Hkv & 1) || H % Hkv)
    return DZ_ERR_ARG;
  if (ldo < 3LL * H * 128 || (reinterpret_cast<uintptr_t>(cs) & 15)) return DZ_ERR_ALIGN;
  Gemm2Args r{};
  r.rope_cs = cs; r.rope_L = L; r.rope_pos0 = pos0; r.rope_n_pos = n_pos; r.rope_H = H; r.rope_Hkv = Hkv;
  return gemm2_launch(A, lda, W, ldw, out, ldo, nullptr, nullptr, 0, M, (H + 2 * Hkv) * 128, K, 4, 0, 1.0f, err,
                      stream, &r);
}

static int gemm2_launch(const void* A, long long lda, const void* W, long long ldw, void* out,
                        long long ldo, const void* bias, const void* residual, long long ldr,
                        int M, int N, int K, int act, int out_fp32, float out_scale,
                        uint32_t* err, cudaStream_t stream, const Gemm2Args* rope) {
  if (!A || !W || !out || M <= 0 || N <= 0 || K <= 0) return DZ_ERR_ARG;
  if ((K & 7) || (lda & 7) || (ldw & 7)) return DZ_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return DZ_ERR_ALIGN;
  int esz = out_fp32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(out) & 15) || ((ldo * esz) & 15)) return DZ_ERR_ALIGN;
  if (bias && (reinterpret_cast<uintptr_t>(bias) & 15)) return DZ_ERR_ALIGN;
  if (residual && ((reinterpret_cast<uintptr_t>(residual) & 15) || (ldr & 7))) return DZ_ERR_ALIGN;
  // act 3: W = gate rows | up rows (N / 2 each), out [M, N / 2] = silu(A gate^T) * (A up^T), bf16, no bias
  if (act == 3 && ((N % G2_BN) || bias || residual || out_fp32 || out_scale != 1.0f || ldo < N / 2))
    return DZ_ERR_ARG;
  Gemm2Args a{};
  a.M = M; a.N = N; a.K = K;
  a.out = out; a.ldo = ldo;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  a.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  a.ldr = ldr; a.act = act; a.out_fp32 = out_fp32; a.out_scale = out_scale; a.err = err;
  // 256-bit stores need 32-byte aligned rows (DIZO_GEMM_ST256=0 keeps the 128-bit ones, for measurements)
  static const bool st256 = [] { const char* e = getenv("DIZO_GEMM_ST256"); return !(e && e[0] == '0'); }();
  a.wide_store = st256 && !out_fp32 && !(reinterpret_cast<uintptr_t>(out) & 31) && !(ldo & 15);
  a.wide_residual = st256 && residual && !(reinterpret_cast<uintptr_t>(residual) & 31) && !(ldr & 15);
  if (rope) {
    a.rope_cs = rope->rope_cs; a.rope_L = rope->rope_L; a.rope_pos0 = rope->rope_pos0;
    a.rope_n_pos = rope->rope_n_pos; a.rope_H = rope->rope_H; a.rope_Hkv = rope->rope_Hkv;
  }
  a.num_m = (M + G2_BM - 1) / G2_BM;
  a.num_n = (N + G2_BN - 1) / G2_BN;
  // M tiles per rasterisation group: a group's A tiles stay in L2 while its W tiles stream once
  static const int group_env = [] { const char* e = getenv("DIZO_GEMM_GROUP_M"); return e ? atoi(e) : 0; }();
  // 16 while the group's A tiles (256 x K bf16 each) stay within about 48 MB of L2 (K = 5120: +1 % over 8 on the
  // QKV / fc1 / out_proj shapes), else 8 (K = 20480: 16 measured -0.8 %, 4 measured -5 %, 32 is worse everywhere);
  // DIZO_GEMM_GROUP_M overrides for measurements
  int gm = (long long)16 * G2_BM * K * 2 > (48LL << 20) ? 8 : 16;
  if (group_env > 0) gm = group_env;
  a.group_m = a.num_m < gm ? a.num_m : gm;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_bf16_2d(&tmA, A, M, K, lda, 128, G2_BK, true);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tmB, W, N, K, ldw, G2_BN / 2, G2_BK, true);
  if (rc) return rc;
  static PerDeviceFlag configured;
  if (int rc_cfg = ensure_dyn_smem(configured, gemm2_bf16_tn_kernel, G2_SMEM)) return rc_cfg;
  int tiles = a.num_m * a.num_n;
  static int max_clusters = 0;
  if (!max_clusters) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count() & ~1);
    cfg.blockDim = dim3(G2_THREADS);
    cfg.dynamicSmemBytes = G2_SMEM;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm2_bf16_tn_kernel, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = sm_count() / 2;
    }
    max_clusters = n < sm_count() / 2 ? n : sm_count() / 2;
  }
  int clusters = max_clusters;
  if (tiles < clusters) clusters = tiles;
  gemm2_bf16_tn_kernel<<<clusters * 2, G2_THREADS, G2_SMEM, stream>>>(tmA, tmB, a);
  return cuda_rc(cudaGetLastError());
}
