// Persistent bf16 GEMM for sm_100a:  out[M,N] = epilogue( A[M,K] * W[N,K]^T ).
//
// Both operands are K-major (activations row-major, weights in the nn.Linear
// [out_features, in_features] layout), so a tile of either is a TMA box of
// 64 bf16 (128 bytes) x rows with the 128-byte swizzle, which is exactly the
// canonical K-major UMMA operand layout.
//
// One CTA per SM, 6 warps, warp-specialised:
//   warp 0   : TMA producer (one elected lane), STAGES-deep ring of {A 128x64, W BNx64}
//   warp 1   : allocates TMEM, one elected lane issues tcgen05.mma (128 x BN x 16 per
//              instruction, fp32 accumulators in TMEM), commits to the ring's "empty"
//              barriers and to the accumulator's "full" barrier
//   warps 2-5: epilogue; each warp owns one 32-lane TMEM quadrant, a thread owns one
//              output row.  tcgen05.ld -> bias / activation / residual -> bf16 or fp32
//              stores, or (EPI_LSE) a per-row online log-sum-exp over the tile's
//              columns so the [rows, vocab] logits never reach memory.
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue of
// tile i overlaps the main loop of tile i+1.
//
// Replaces the cuBLAS calls behind nn.Linear in the reference's OPT forward
// (large_models/ht_opt.py:178-197, :274, :356-359) and the lm_head + log_softmax
// (large_models/ht_opt.py:956, large_models/trainer.py:1469-1489).
#include "common.cuh"
#include "host_util.h"

namespace dz {

constexpr int G_BM = 128;
constexpr int G_BK = 64;
constexpr int G_THREADS = 192;

enum { EPI_STORE = 0, EPI_LSE = 1 };
enum { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2 };

struct GemmArgs {
  int M, N, K;
  int num_m, num_n, group_m;
  // EPI_STORE
  void* out;            // bf16 or fp32 [M, ldo]
  long long ldo;
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldr] or null
  long long ldr;
  const __nv_bfloat16* mask;      // [M, ldm] or null: the result is zeroed where mask <= 0 (ReLU backward)
  long long ldm;
  int act;
  int out_fp32;
  float out_scale;      // multiplies (acc + bias) before activation/residual
  // EPI_LSE
  const int* targets;   // [M] column whose logit is wanted, or null
  float* part_max;      // [M, num_n]
  float* part_sum;      // [M, num_n]
  float* tgt_logit;     // [M]
  uint32_t* err;
};

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = G_BM * G_BK * 2;
  static constexpr int B_BYTES = BN * G_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024;  // + alignment slack
};

__device__ __forceinline__ void tile_coords(int tile, const GemmArgs& p, int& mb, int& nb) {
  // Grouped rasterisation: consecutive tiles walk down group_m row blocks of the same
  // column block, so the tiles resident at one time share A rows and W columns in L2.
  int tiles_per_group = p.group_m * p.num_n;
  int g = tile / tiles_per_group;
  int first_m = g * p.group_m;
  int gm = min(p.group_m, p.num_m - first_m);
  int r = tile - g * tiles_per_group;
  mb = first_m + r % gm;
  nb = r / gm;
}

// B_MN = false: W is [N, K] row-major (out = A W^T, both operands K-major).
// B_MN = true : W is [K, N] row-major (out = A W, the data-gradient form dX = dY W of a linear
//               layer): the B operand is MN-major, staged as 64-column panels of [64 k-rows][128 B].
template <int BN, int STAGES, int EPI, bool B_MN = false>
__global__ void __launch_bounds__(G_THREADS, 1)
gemm_bf16_tn_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmArgs p) {
  using S = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[STAGES];
  __shared__ __align__(8) uint64_t bar_empty[STAGES];
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile int s_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int num_tiles = p.num_m * p.num_n;
  const int num_kb = (p.K + G_BK - 1) / G_BK;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_acc_full[a]), 1);
      mbar_init(smem_u32(&bar_acc_empty[a]), 4);
    }
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&s_tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mb, nb;
        tile_coords(tile, p, mb, nb);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1, &s_abort, p.err, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          uint32_t full = smem_u32(&bar_full[stage]);
          uint32_t a_dst = smem_base + stage * S::STAGE_BYTES;
          uint32_t b_dst = a_dst + S::A_BYTES;
          mbar_arrive_expect_tx(full, S::STAGE_BYTES);
          tma_load_2d(a_dst, &tmA, full, kb * G_BK, mb * G_BM);
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(b_dst + c * (G_BK * 128), &tmB, full, nb * BN + c * 64, kb * G_BK);
          } else {
            tma_load_2d(b_dst, &tmB, full, kb * G_BK, nb * BN);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(G_BM, BN, 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(smem_u32(&bar_acc_empty[acc]), acc_phase ^ 1, &s_abort, p.err,
                       ERR_WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &s_abort, p.err, ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          uint32_t a_src = smem_base + stage * S::STAGE_BYTES;
          uint32_t b_src = a_src + S::A_BYTES;
          uint64_t a_desc = umma_desc_k_sw128(a_src);
          uint64_t b_desc = umma_desc_k_sw128(b_src);
#pragma unroll
          for (int k = 0; k < G_BK / 16; ++k) {
            // advancing 16 bf16 along K inside the 128-byte swizzle row = +32 bytes
            if (B_MN) {
              // 16 k-rows = two 8-row groups of 1024 bytes; 64-column panels are G_BK*128 bytes apart
              umma_bf16_ss(d_tmem, a_desc + 2 * k, umma_desc_mn_sw128(b_src + k * 2048, G_BK * 128, 1024),
                           idesc, (kb | k) != 0);
            } else {
              umma_bf16_ss(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
            }
          }
          umma_commit(smem_u32(&bar_empty[stage]));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(smem_u32(&bar_acc_full[acc]));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int mb, nb;
      tile_coords(tile, p, mb, nb);
      if (!mbar_wait(smem_u32(&bar_acc_full[acc]), acc_phase, &s_abort, p.err, ERR_WAIT_TMEM_FULL))
        break;
      tc_fence_after();
      const long long row = (long long)mb * G_BM + row_in_tile;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);

      float run_max = -INFINITY, run_sum = 0.f;
      int tgt = -1;
      if (EPI == EPI_LSE) tgt = (row_ok && p.targets) ? p.targets[row] : -1;

#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = nb * BN + c * 32;
        if (col0 >= p.N) continue;  // whole chunk past the edge (warp-uniform)
        if (EPI == EPI_STORE) {
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
          if (p.act == ACT_RELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
          } else if (p.act == ACT_GELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
          }
          if (row_ok) {
            if (p.mask) {
              const __nv_bfloat16* mp = p.mask + row * p.ldm + col0;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N && !(__bfloat162float(mp[j]) > 0.f)) v[j] = 0.f;
            }
            if (p.residual) {
              const __nv_bfloat16* rp = p.residual + row * p.ldr + col0;
              if (full_chunk) {
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
                uint4* op4 = reinterpret_cast<uint4*>(op);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  uint4 o;
                  o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
                  o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
                  o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
                  o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
                  if (DZ_STORE_OK(op4 + q, 16)) op4[q] = o;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < p.N && DZ_STORE_OK(op + j, 2)) op[j] = __float2bfloat16(v[j]);
              }
            }
          }
        } else {
          // EPI_LSE: online (max, sum exp) over this tile's valid columns + target pick-up
          float cmax = -INFINITY;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float x = (col0 + j < p.N) ? __uint_as_float(r[j]) * p.out_scale : -INFINITY;
            r[j] = __float_as_uint(x);
            cmax = fmaxf(cmax, x);
          }
          float nmax = fmaxf(run_max, cmax);
          float s = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) s += __expf(__uint_as_float(r[j]) - nmax);
          run_sum = run_sum * __expf(run_max - nmax) + s;
          run_max = nmax;
          if (tgt >= col0 && tgt < col0 + 32) {
            float t = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j == tgt) t = __uint_as_float(r[j]);
            p.tgt_logit[row] = t;
          }
        }
      }
      if (EPI == EPI_LSE && row_ok) {
        p.part_max[row * p.num_n + nb] = run_max;
        p.part_sum[row * p.num_n + nb] = run_sum;
      }
      // accumulator drained: hand it back to the MMA issuer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[acc]));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // ---------------------------------------------------------------- tear-down
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (s_abort) {
      // error path: give copies and MMAs still in flight time to land before TMEM goes
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, int STAGES, int EPI, bool B_MN = false>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmArgs& a,
                       cudaStream_t stream) {
  using S = GemmSmem<BN, STAGES>;
  auto kern = gemm_bf16_tn_kernel<BN, STAGES, EPI, B_MN>;
  static PerDeviceFlag configured;
  if (int rc_cfg = ensure_dyn_smem(configured, kern, S::TOTAL)) return rc_cfg;
  a.num_m = (a.M + G_BM - 1) / G_BM;
  a.num_n = (a.N + BN - 1) / BN;
  a.group_m = a.num_m < 16 ? a.num_m : 16;
  int tiles = a.num_m * a.num_n;
  int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, G_THREADS, S::TOTAL, stream>>>(tmA, tmB, a);
  return cuda_rc(cudaGetLastError());
}

static int check_common(const void* A, const void* W, int M, int N, int K, long long lda,
                        long long ldw) {
  if (!A || !W || M <= 0 || N <= 0 || K <= 0) return DZ_ERR_ARG;
  if ((K & 7) || (lda & 7) || (ldw & 7)) return DZ_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    return DZ_ERR_ALIGN;
  return DZ_OK;
}

}  // namespace dz

using namespace dz;
DZ_DEBUG_TU(gemm1)

// out[M,N] = act((A W^T + bias) * out_scale) + residual.  bf16 inputs; out is bf16 or fp32.
// tile_n: 0 = choose, 128 or 256.
extern "C" int dz_gemm_bf16_tn(const void* A, long long lda, const void* W, long long ldw, void* out,
                               long long ldo, const void* bias, const void* residual, long long ldr,
                               int M, int N, int K, int act, int out_fp32, float out_scale,
                               int tile_n, uint32_t* err, cudaStream_t stream) {
  int rc = check_common(A, W, M, N, K, lda, ldw);
  if (rc) return rc;
  if (!out) return DZ_ERR_ARG;
  // vector stores in the epilogue need 16-byte aligned rows
  int esz = out_fp32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(out) & 15) || ((ldo * esz) & 15)) return DZ_ERR_ALIGN;
  if (bias && (reinterpret_cast<uintptr_t>(bias) & 15)) return DZ_ERR_ALIGN;
  if (residual && ((reinterpret_cast<uintptr_t>(residual) & 15) || (ldr & 7))) return DZ_ERR_ALIGN;
  GemmArgs a{};
  a.M = M; a.N = N; a.K = K;
  a.out = out; a.ldo = ldo;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  a.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  a.ldr = ldr; a.act = act; a.out_fp32 = out_fp32; a.out_scale = out_scale; a.err = err;
  if (tile_n == 0) {
    // 256-wide tiles unless that leaves most SMs idle
    long long tiles256 = (long long)((M + G_BM - 1) / G_BM) * ((N + 255) / 256);
    tile_n = (tiles256 < sm_count() && N > 128) ? 128 : 256;
  }
  CUtensorMap tmA, tmB;
  rc = make_tmap_bf16_2d(&tmA, A, M, K, lda, G_BM, G_BK, true);
  if (rc) return rc;
  if (tile_n == 128) {
    rc = make_tmap_bf16_2d(&tmB, W, N, K, ldw, 128, G_BK, true);
    if (rc) return rc;
    return launch_gemm<128, 6, EPI_STORE>(tmA, tmB, a, stream);
  }
  rc = make_tmap_bf16_2d(&tmB, W, N, K, ldw, 256, G_BK, true);
  if (rc) return rc;
  return launch_gemm<256, 4, EPI_STORE>(tmA, tmB, a, stream);
}

// out[M,N] = (A W) masked + residual with W [K, N] row-major: the data gradient dX = dY W of a
// linear layer whose weight is stored [out_features, in_features], read in place (no transposed
// copy).  mask [M, ldm] (optional): entries whose mask is <= 0 become 0 (the ReLU backward of the
// layer below, fused); residual [M, ldr] (optional) is added afterwards (gradient accumulation).
// Replaces the autograd matmul backward of large_models/ht_opt.py:178-197, :356-359 in the
// first-order gamma search (large_models/trainer.py:714-741).
extern "C" int dz_gemm_bf16_nn(const void* A, long long lda, const void* W, long long ldw, void* out,
                               long long ldo, const void* residual, long long ldr, const void* mask,
                               long long ldm, int M, int N, int K, int out_fp32, uint32_t* err,
                               cudaStream_t stream) {
  if (!A || !W || !out || M <= 0 || N <= 0 || K <= 0) return DZ_ERR_ARG;
  if ((K & 7) || (N & 7) || (lda & 7) || (ldw & 7)) return DZ_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return DZ_ERR_ALIGN;
  int esz = out_fp32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(out) & 15) || ((ldo * esz) & 15)) return DZ_ERR_ALIGN;
  if (residual && ((reinterpret_cast<uintptr_t>(residual) & 15) || (ldr & 7))) return DZ_ERR_ALIGN;
  GemmArgs a{};
  a.M = M; a.N = N; a.K = K;
  a.out = out; a.ldo = ldo;
  a.residual = reinterpret_cast<const __nv_bfloat16*>(residual); a.ldr = ldr;
  a.mask = reinterpret_cast<const __nv_bfloat16*>(mask); a.ldm = ldm;
  a.act = ACT_NONE; a.out_fp32 = out_fp32; a.out_scale = 1.0f; a.err = err;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_bf16_2d(&tmA, A, M, K, lda, G_BM, G_BK, true);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tmB, W, K, N, ldw, G_BK, 64, true);      // box: 64 k-rows x 64 columns
  if (rc) return rc;
  return launch_gemm<256, 4, EPI_STORE, true>(tmA, tmB, a, stream);
}

// Fused logits + log-sum-exp partials: for every row r of A, over columns n of W:
//   part_max[r, j], part_sum[r, j] = online (max, sum exp(x - max)) over column tile j,
//   x = (A W^T)[r, n] * out_scale;  tgt_logit[r] = x[r, targets[r]] (if targets given).
// The number of column tiles is ceil(N / 256); the caller combines them
// (dz_lse_combine).  Nothing of size [M, N] is written.
extern "C" int dz_gemm_bf16_tn_lse(const void* A, long long lda, const void* W, long long ldw,
                                   const int* targets, float* part_max, float* part_sum,
                                   float* tgt_logit, int M, int N, int K, float out_scale,
                                   uint32_t* err, cudaStream_t stream) {
  int rc = check_common(A, W, M, N, K, lda, ldw);
  if (rc) return rc;
  if (!part_max || !part_sum || (targets && !tgt_logit)) return DZ_ERR_ARG;
  GemmArgs a{};
  a.M = M; a.N = N; a.K = K;
  a.targets = targets; a.part_max = part_max; a.part_sum = part_sum; a.tgt_logit = tgt_logit;
  a.out_scale = out_scale; a.err = err;
  CUtensorMap tmA, tmB;
  rc = make_tmap_bf16_2d(&tmA, A, M, K, lda, G_BM, G_BK, true);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tmB, W, N, K, ldw, 256, G_BK, true);
  if (rc) return rc;
  return launch_gemm<256, 4, EPI_LSE>(tmA, tmB, a, stream);
}

extern "C" int dz_gemm_lse_num_tiles(int N) { return (N + 255) / 256; }

// ------------------------------------------------------------------------------------------
// Allocation-free token log-probabilities (see dizo_noalloc.h).
// ------------------------------------------------------------------------------------------
#include "dizo_noalloc.h"

namespace {

constexpr int NA_TILES = (DZ_NOALLOC_MAX_VOCAB + 255) / 256;
constexpr size_t NA_PART = (size_t)DZ_NOALLOC_MAX_ROWS * NA_TILES;       // floats per partial array
constexpr size_t NA_FLOATS = 2 * NA_PART + DZ_NOALLOC_MAX_ROWS;          // max, sum, target logit

// Scratch owned by the library.  In host code this name is only a handle for
// cudaGetSymbolAddress, never a device address to hand to a kernel.
static __device__ __align__(256) float g_noalloc_scratch[NA_FLOATS];

constexpr int NA_MAX_DEVICES = 64;
static float* g_noalloc_ptr[NA_MAX_DEVICES] = {};

__global__ void noalloc_combine_kernel(const float* __restrict__ part_max,
                                       const float* __restrict__ part_sum,
                                       const float* __restrict__ tgt_logit, int num_tiles, int rows,
                                       float* __restrict__ logprob) {
  int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const float* pm = part_max + (long long)r * num_tiles;
  const float* ps = part_sum + (long long)r * num_tiles;
  float m = -INFINITY;
  for (int j = 0; j < num_tiles; ++j) m = fmaxf(m, pm[j]);
  float s = 0.f;
  for (int j = 0; j < num_tiles; ++j) s += ps[j] * expf(pm[j] - m);
  logprob[r] = tgt_logit[r] - (m + logf(s));
}

}  // namespace

extern "C" int dz_token_logprobs_noalloc(const void* A, long long lda, const void* W, long long ldw,
                                         const int* targets, float* out_logprob, int M, int N, int K,
                                         float scale, uint32_t* err, cudaStream_t stream) {
  int rc = check_common(A, W, M, N, K, lda, ldw);
  if (rc) return rc;
  if (!targets || !out_logprob) return DZ_ERR_ARG;
  if (M > DZ_NOALLOC_MAX_ROWS || N > DZ_NOALLOC_MAX_VOCAB) return DZ_ERR_TOO_LARGE;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_rc(e);
  if (dev < 0 || dev >= NA_MAX_DEVICES) return DZ_ERR_ARG;
  if (!g_noalloc_ptr[dev]) {
    // set-up, once per device, with that device current
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess) return cuda_rc(e);
    g_noalloc_ptr[dev] = p;
  }
  float* part_max = g_noalloc_ptr[dev];
  float* part_sum = part_max + NA_PART;
  float* tgt = part_sum + NA_PART;
  // the gold logit of a row is only written when its target lies inside [0, N): start clean
  e = cudaMemsetAsync(tgt, 0, sizeof(float) * M, stream);
  if (e != cudaSuccess) return cuda_rc(e);
  GemmArgs a{};
  a.M = M; a.N = N; a.K = K;
  a.targets = targets; a.part_max = part_max; a.part_sum = part_sum; a.tgt_logit = tgt;
  a.out_scale = scale; a.err = err;
  CUtensorMap tmA, tmB;
  rc = make_tmap_bf16_2d(&tmA, A, M, K, lda, G_BM, G_BK, true);
  if (rc) return rc;
  rc = make_tmap_bf16_2d(&tmB, W, N, K, ldw, 256, G_BK, true);
  if (rc) return rc;
  rc = launch_gemm<256, 4, EPI_LSE>(tmA, tmB, a, stream);
  if (rc) return rc;
  const int tiles = (N + 255) / 256;
  noalloc_combine_kernel<<<(M + 127) / 128, 128, 0, stream>>>(part_max, part_sum, tgt, tiles, M,
                                                             out_logprob);
  return cuda_rc(cudaGetLastError());
}
