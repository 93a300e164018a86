// GEMM fused with its collective over peer memory (NVLink / NVSwitch), one launch:
//
//   out = epilogue( A[M,K] * W[N,K]^T )       tcgen05 / TMEM / TMA, as gemm_sm100.cu
//
// plus any of
//   * PUSH role (four extra warps in the first n_push CTAs): copy a block of local rows into every peer's
//     staging buffer with plain posted stores (all-gather by push), optionally transforming it on
//     the way: theta + c * z(seed) regenerated from Philox for the pushed shard (FSDP parameter
//     all-gather fused with the perturbation - the owner perturbs its shard once, nobody
//     materialises z).  The push warps of CTA b move slice b of the rows while the producer, MMA
//     and epilogue warps of the same CTA run GEMM tiles: a tcgen05 GEMM leaves the issue slots and
//     the load/store path of its SM almost idle, so the transfer rides along without taking SMs
//     away from the tensor-core work (dedicating whole CTAs to it cost 16 of 148 SMs).  How many
//     CTAs push is the host's choice per launch, from the bytes to move and the time the GEMM
//     gives them: posted stores from all 148 SMs saturate NVLink within a fraction of the launch
//     and the back-pressure then stalls the TMA loads of every GEMM (measured on 8 GPUs), so the
//     host limits the pushing CTAs and gives them a smaller share of the tiles, or none
//     (`join_tiles`; their tiles sit at the end of the tile order).  When a CTA has pushed its slice it
//     fences at system scope; the last one raises the `ready` flag of this rank at every peer.
//   * GATHERED OPERAND: rows of A (tensor parallel: sequence-sharded activations) or of W
//     (FSDP: row-sharded weights) arrive from peers in this rank's staging buffer; the TMA
//     producer polls the source rank's `ready` flag (bounded) before its first load of rows
//     that rank owns, and tiles are visited own-rows-first, so math on what is already here
//     overlaps the arrival of the rest.
//   * PUSH EPILOGUE (GEMM -> reduce-scatter): every output tile is stored straight into the
//     staging slot [this rank] of the rank that owns those rows; after the last tile the
//     last CTA raises this rank's `partials ready` flag at every owner
//     (dz_rs_reduce_layernorm in comm_kernels.cu is the owner side).
//   * ACK: when the GEMM has consumed a gathered operand, the last CTA tells every peer that
//     the staging buffer may be overwritten; a pusher waits (bounded) for those acks first.
//
// No load in this file uses cluster multicast and nothing is loaded from a peer: remote data
// always arrives by the peer's stores into local memory, then is read with local TMA loads.
// All waits are bounded and report through the error word.
#include "common.cuh"
#include "cluster2sm.cuh"
#include "host_util.h"
#include "philox.cuh"

namespace dz {

constexpr int CG_BM = 128;
constexpr int CG_BN = 256;
constexpr int CG_BK = 64;
constexpr int CG_STAGES_PUSH = 4;   // ring depth with the reduce-scatter epilogue (plus 32 KB of row staging)
constexpr int CG_STAGES_PLAIN = 4;
constexpr int CG_GEMM_THREADS = 192;   // warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 epilogue
constexpr int CG_PUSH_THREADS = 128;   // warps 6-9: the push role
constexpr int CG_THREADS = CG_GEMM_THREADS + CG_PUSH_THREADS;
constexpr int CG_TABLE_BYTES = GAUSS_BINS * 4;   // plain copy of the inverse-CDF pairs for perturbing pushes
constexpr int CG_A_BYTES = CG_BM * CG_BK * 2;
constexpr int CG_B_BYTES = CG_BN * CG_BK * 2;
constexpr int CG_STAGE_BYTES = CG_A_BYTES + CG_B_BYTES;
constexpr int CG_OUT_STAGE_BYTES = 4 * 32 * 256;                // per epilogue warp: 32 rows x 128 bf16 columns
// behind the operand ring: the row staging of the push epilogue, or the table of a perturbing push
// (never both in one launch)
constexpr int CG_SMEM_PUSH = CG_STAGES_PUSH * CG_STAGE_BYTES + CG_OUT_STAGE_BYTES + 1024;
constexpr int CG_SMEM_PLAIN = CG_STAGES_PLAIN * CG_STAGE_BYTES + CG_TABLE_BYTES + 1024;
static_assert(CG_STAGES_PUSH == CG_STAGES_PLAIN, "one kernel instantiation expected");
static_assert(CG_TABLE_BYTES <= CG_OUT_STAGE_BYTES, "the table must fit where the row staging sits");
constexpr uint32_t CG_TMEM_COLS = 2 * CG_BN;
constexpr int CG_MAX_WORLD = 16;
constexpr int CG_MAXC = 16;            // progress chunks per source in a gathered operand
constexpr int CG_PUSH_UNROLL = 8;

struct CommGemmArgs {
  // ---- GEMM
  int M, N, K;
  int num_m, num_n;
  void* out;                     // local output (ignored with push_out)
  long long ldo;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  long long ldr;
  int act, out_fp32;
  float out_scale;
  int wide_store;                // local bf16 output rows are 32-byte aligned: 256-bit stores
  // ---- gathered operand: 0 none, 1 = rows of A come from peers, 2 = rows of W come from peers
  int gather;
  int rows_per_src;              // rows owned by each source rank
  int src_period;                // W rows repeat their ownership pattern every src_period rows
                                 // (fused q|k|v: d); 0 = no repetition
  int wait_self;                 // own rows are also produced by this launch's push role
  int chunk_tiles;               // gather 1: row tiles per progress chunk of a source (0 = one chunk)
  int join_tiles;                // tiles at the end of the order that the pushing CTAs multiply (< 0: none)
  const uint32_t* ready_flags;   // local [world][CG_MAXC]: flag[s][c] >= ready_epoch once rank s has
                                 // pushed chunk c of its rows (unchunked pushes use c = 0 only)
  uint32_t ready_epoch;
  // ---- ack of a consumed gathered operand
  uint32_t* const* ack_ptrs;     // per rank: pointer to its [world] ack words
  uint32_t ack_epoch;
  // ---- push epilogue (reduce-scatter)
  int push_out;
  void* const* out_ptrs;         // per owner rank: base of its [world][rows_per_owner][ldo] staging
  long long out_slot_stride;     // elements between the slots of two source ranks
  int rows_per_owner;
  uint32_t* const* rs_flag_ptrs; // per rank: its [world] "partials ready" words
  uint32_t rs_epoch;
  // ---- push role
  int n_push;                    // CTAs whose push warps are active (the first n_push; 0 = no push)
  int push_nseg;                 // 1..3 row segments of equal shape (e.g. the q, k, v shards)
  const __nv_bfloat16* push_src[3]; // local rows [push_rows, push_cols], row stride push_ld
  long long push_ld;
  long long push_rows, push_cols;
  void* const* push_dst_ptrs;    // per rank: base of the destination buffer
  long long push_dst_ld;
  long long push_dst_row0[3];    // first destination row of each segment (same in every peer)
  int push_to_self;
  long long push_chunk_rows;     // plain copies: rows per progress chunk (0 = the whole push)
  uint32_t* const* push_flag_ptrs;   // per rank: its [world][CG_MAXC] ready words
  uint32_t push_epoch;
  const uint32_t* push_wait_acks;    // local [world] ack words to wait for before overwriting
  uint32_t push_wait_epoch;          // (0 = do not wait)
  // perturbation of the pushed rows
  int push_perturb;
  unsigned long long push_seed;
  float push_coef;
  int push_tensor_id[3];
  long long push_elem_base[3];   // index of push_src[s][0,0] inside the full tensor
  const uint32_t* gauss_table;
  // ---- bookkeeping
  int rank, world;
  unsigned int* counters;        // local [2 + CG_MAXC]: pushers done, gemm CTAs done, pushers done per
                                 // progress chunk (all monotonic)
  unsigned int push_target, gemm_target;
  uint32_t* err;
};

__device__ __forceinline__ void cg_st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t cg_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool cg_wait_flag(const uint32_t* p, uint32_t epoch, volatile int* abort_flag,
                                             uint32_t* err) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while ((int32_t)(cg_ld_acquire_sys(p) - epoch) < 0) {
    if ((++spins & 0x3f) == 0) {
      if (abort_flag && *abort_flag) return false;
      uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > DZ_WAIT_TIMEOUT_NS) {
        if (abort_flag) *abort_flag = 1;
        if (err) atomicCAS(err, 0u, (uint32_t)ERR_WAIT_PEER | (blockIdx.x << 8));
        return false;
      }
    }
    __nanosleep(100);
  }
  return true;
}

// Tiles are visited source by source, own rows first.
// (`bm`: rows of a tile - 128 for the one-SM kernel, 256 for the two-SM kernel)
__device__ __forceinline__ void cg_tile_coords(int tile, const CommGemmArgs& p, const int bm, int& mb, int& nb) {
  if (p.gather == 1) {
    // own rows first; then chunk by chunk (every source pushes its chunk c to all ranks before chunk
    // c+1, so this is the order in which the rows arrive).  Inside the own block and inside a chunk
    // the walk is column-major - all row tiles of the group for one 256-column block of W, then the
    // next block - so the CTAs in flight share a few W tiles and the group's A rows instead of
    // streaming the whole of W (which exceeds L2 at small world sizes) once per row tile.
    const int mbs = p.rows_per_src / bm;             // row tiles per source
    const int per_src = mbs * p.num_n;
    if (tile < per_src) {
      mb = p.rank * mbs + tile % mbs;
      nb = tile / mbs;
    } else {
      const int ct = p.chunk_tiles > 0 ? p.chunk_tiles : mbs;
      const int rows_c = ct * (p.world - 1);         // row tiles of one chunk over all sources
      const int per_c = rows_c * p.num_n;
      int t = tile - per_src;
      const int c = t / per_c;
      t -= c * per_c;
      nb = t / rows_c;
      const int rr = t - nb * rows_c;
      const int s = rr / ct + 1;
      const int src = (p.rank + s) % p.world;
      mb = src * mbs + c * ct + (rr - (s - 1) * ct);
    }
  } else {
    int gm = p.num_m < 16 ? p.num_m : 16;
    int tiles_per_group = gm * p.num_n;
    int g = tile / tiles_per_group;
    int first_m = g * gm;
    int gmm = min(gm, p.num_m - first_m);
    int r = tile - g * tiles_per_group;
    mb = first_m + r % gmm;
    nb = r / gmm;
  }
}

// Barrier of the push warps only (named barrier 1); the GEMM warps never wait on it.
__device__ __forceinline__ void cg_push_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(CG_PUSH_THREADS) : "memory");
}

// Executed by the CG_PUSH_THREADS push threads of every CTA; `pt` is the thread's index among them,
// slice `blockIdx.x` of `n_push` equal slices of the rows is this CTA's share.
__device__ __forceinline__ void cg_push_role(const CommGemmArgs& p, uint8_t* table_smem, const int pt) {
  const int n_slices = p.n_push;
  __shared__ int s_go;
  __shared__ int s_first_idle;     // first chunk counter this launch leaves untouched
  // stage the inverse-CDF table when the pushed rows are perturbed
  const char* tab = reinterpret_cast<const char*>(table_smem);
  if (p.push_perturb) {
    // the plain 4 KB table (the lane-replicated 128 KB copy of the sweep kernel does not fit beside the
    // GEMM's operand ring; the bank conflicts cost nothing here, the transfer is NVLink-bound)
    for (int i = pt; i < GAUSS_BINS; i += CG_PUSH_THREADS)
      reinterpret_cast<uint32_t*>(table_smem)[i] = __ldg(p.gauss_table + i);
  }
  if (pt == 0) { s_go = 1; s_first_idle = 0; }
  cg_push_sync();
  // the peers must have consumed what this buffer held before
  if (p.push_wait_epoch != 0 && pt < p.world && pt != p.rank) {
    if (!cg_wait_flag(p.push_wait_acks + pt, p.push_wait_epoch, nullptr, p.err)) s_go = 0;
  }
  cg_push_sync();
  if (s_go) {
    const long long vec_per_row = p.push_cols >> 3;
    const long long seg_total = p.push_rows * vec_per_row;
    const long long total = seg_total * p.push_nseg;
    const long long per = (total + n_slices - 1) / n_slices;
    const long long v0 = (long long)blockIdx.x * per;
    const long long v1 = min(v0 + per, total);
    if (!p.push_perturb) {
      // Plain copy, chunk by chunk: `push_chunk_rows` rows of every segment go to all destinations
      // (each 16-byte vector is loaded once and stored to every peer, nearest consumer first:
      // rank d reads the rows of d+1, d+2, ... in that order), then that chunk's ready flag goes up
      // everywhere, so consumers multiply chunk c while chunk c+1 travels.
      const long long crows = p.push_chunk_rows > 0 ? p.push_chunk_rows : p.push_rows;
      const int nchunks = (int)((p.push_rows + crows - 1) / crows);
      for (int c = 0; c < nchunks; ++c) {
        const long long row_lo = (long long)c * crows;
        const long long rows_c = min(crows, p.push_rows - row_lo);
        const long long seg_c = rows_c * vec_per_row;
        const long long total_c = seg_c * p.push_nseg;
        const long long per_c = (total_c + n_slices - 1) / n_slices;
        const long long c0 = (long long)blockIdx.x * per_c;
        const long long c1 = min(c0 + per_c, total_c);
        for (long long base = c0; base < c1; base += (long long)CG_PUSH_THREADS * CG_PUSH_UNROLL) {
          uint4 raw[CG_PUSH_UNROLL];
          long long doff[CG_PUSH_UNROLL];
          bool live[CG_PUSH_UNROLL];
#pragma unroll
          for (int u = 0; u < CG_PUSH_UNROLL; ++u) {
            const long long vv = base + (long long)u * CG_PUSH_THREADS + pt;
            live[u] = vv < c1;
            if (live[u]) {
              const int seg = (int)(vv / seg_c);
              const long long v = vv - seg * seg_c;
              const long long r = row_lo + v / vec_per_row, cc = (v % vec_per_row) << 3;
              raw[u] = *reinterpret_cast<const uint4*>(p.push_src[seg] + r * p.push_ld + cc);
              doff[u] = (p.push_dst_row0[seg] + r) * p.push_dst_ld + cc;
            }
          }
          for (int sdst = 1; sdst <= p.world; ++sdst) {
            const int d = (p.rank - sdst + 2 * p.world) % p.world;
            if (d == p.rank && !p.push_to_self) continue;
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.push_dst_ptrs[d]);
#pragma unroll
            for (int u = 0; u < CG_PUSH_UNROLL; ++u)
              if (live[u] && DZ_STORE_OK(dst + doff[u], 16)) *reinterpret_cast<uint4*>(dst + doff[u]) = raw[u];
          }
        }
        __threadfence_system();
        cg_push_sync();
        if (pt == 0) {
          unsigned int old = atomicAdd(p.counters + 2 + c, 1u);
          if (old + 1u == p.push_target) {
            __threadfence_system();
            for (int d = 0; d < p.world; ++d)
              cg_st_release_sys(p.push_flag_ptrs[d] + p.rank * CG_MAXC + c, p.push_epoch);
          }
        }
      }
      s_first_idle = nchunks;
    } else {
    // Perturbed push: z is generated once per element, then stored to every destination.
    // CG_PUSH_UNROLL independent 16-byte loads per thread are in flight before the first store:
    // a copy loop with one load at a time is bound by local-memory latency, not by NVLink.
    for (long long base = v0; base < v1; base += (long long)CG_PUSH_THREADS * CG_PUSH_UNROLL) {
      uint4 raw[CG_PUSH_UNROLL];
      long long doff[CG_PUSH_UNROLL];
      bool live[CG_PUSH_UNROLL];
#pragma unroll
      for (int u = 0; u < CG_PUSH_UNROLL; ++u) {
        const long long vv = base + (long long)u * CG_PUSH_THREADS + pt;
        live[u] = vv < v1;
        if (live[u]) {
          const int seg = (int)(vv / seg_total);
          const long long v = vv - seg * seg_total;
          const long long r = v / vec_per_row, c = (v - r * vec_per_row) << 3;
          raw[u] = *reinterpret_cast<const uint4*>(p.push_src[seg] + r * p.push_ld + c);
          doff[u] = (p.push_dst_row0[seg] + r) * p.push_dst_ld + c;
        }
      }
      if (p.push_perturb) {
        const uint32_t push_coef_pair = bf16x2_splat(p.push_coef);
#pragma unroll
        for (int u = 0; u < CG_PUSH_UNROLL; ++u) {
          if (!live[u]) continue;
          const long long vv = base + (long long)u * CG_PUSH_THREADS + pt;
          const int seg = (int)(vv / seg_total);
          const long long v = vv - seg * seg_total;
          const long long r = v / vec_per_row, c = (v - r * vec_per_row) << 3;
          const long long e = p.push_elem_base[seg] + r * p.push_cols + c;
          // the same packed bf16 fma as the staging sweep, so a pushed shard equals a swept one bit for bit
          raw[u] = perturb8_packed<2>(tab, p.push_seed, (uint32_t)p.push_tensor_id[seg], (uint32_t)(e >> 3),
                                   push_coef_pair, raw[u]);
        }
      }
      // nearest consumer first: rank d reads the rows of d+1, d+2, ... in that order
      for (int s = 1; s <= p.world; ++s) {
        int d = (p.rank - s + 2 * p.world) % p.world;
        if (d == p.rank && !p.push_to_self) continue;
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.push_dst_ptrs[d]);
#pragma unroll
        for (int u = 0; u < CG_PUSH_UNROLL; ++u)
          if (live[u] && DZ_STORE_OK(dst + doff[u], 16)) *reinterpret_cast<uint4*>(dst + doff[u]) = raw[u];
      }
    }
    }
  }
  __threadfence_system();
  cg_push_sync();
  if (pt == 0) {
    unsigned int old = atomicAdd(p.counters + 0, 1u);
    // the chunk counters this launch did not use stay in step with the common one
    for (int c = s_first_idle; c < CG_MAXC; ++c) atomicAdd(p.counters + 2 + c, 1u);
    if (old + 1u == p.push_target && s_go && p.push_perturb) {
      __threadfence_system();
      for (int d = 0; d < p.world; ++d)
        cg_st_release_sys(p.push_flag_ptrs[d] + p.rank * CG_MAXC, p.push_epoch);
    }
  }
}

// Drain one accumulator of this warp's 32 rows x 256 columns: bias, scale, activation, residual, then the
// store - to the local output, or (push epilogue) staged through shared memory and sent as full-width rows
// to the rank that owns them.  `row` is this lane's output row, `warp_row0` the first row of the warp,
// `t_row` the TMEM address of the warp's lane quadrant in the accumulator.
__device__ __forceinline__ void cg_drain_tile(const CommGemmArgs& p, const uint32_t t_row, const long long row,
                                              const long long warp_row0, const int nb, const int quad,
                                              const int lane, const uint32_t out_stage) {
  const bool row_ok = row < p.M;
  // destination of this row
  __nv_bfloat16* orow_bf = nullptr;
  float* orow_f32 = nullptr;
  if (row_ok) {
    if (p.push_out) {
      int owner = (int)(row / p.rows_per_owner);
      long long lr = row - (long long)owner * p.rows_per_owner;
      orow_bf = reinterpret_cast<__nv_bfloat16*>(p.out_ptrs[owner]) +
                (long long)p.rank * p.out_slot_stride + lr * p.ldo;
    } else if (p.out_fp32) {
      orow_f32 = reinterpret_cast<float*>(p.out) + row * p.ldo;
    } else {
      orow_bf = reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.ldo;
    }
  }
#pragma unroll 1
  for (int c = 0; c < CG_BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(t_row + c * 32, r);
    tmem_ld_wait();
    const int col0 = nb * CG_BN + c * 32;
    if (col0 < p.N) {
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    const bool full_chunk = (col0 + 32 <= p.N);
    if (p.bias) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (full_chunk || col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
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
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (full_chunk || col0 + j < p.N) v[j] += __bfloat162float(rp[j]);
      }
      if (orow_f32) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if ((full_chunk || col0 + j < p.N) && DZ_STORE_OK(orow_f32 + col0 + j, 4)) orow_f32[col0 + j] = v[j];
      } else if (p.push_out) {
        // stage this warp's 32 rows x 128 columns (one half of the tile's width) in its own
        // shared-memory block, 16-byte units XOR-swizzled by the row against bank conflicts
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t unit = (uint32_t)((c & 3) * 4 + q) ^ (uint32_t)(lane & 15);
          const uint32_t addr = out_stage + quad * 8192 + lane * 256 + unit * 16;
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                       "r"(pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1])), "r"(pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3])),
                       "r"(pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5])), "r"(pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]))
                       : "memory");
        }
      } else if (full_chunk) {
        uint4 o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          o[q].x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
          o[q].y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
          o[q].z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
          o[q].w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
        }
        store_row32(orow_bf + col0, o, p.wide_store != 0);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N && DZ_STORE_OK(orow_bf + col0 + j, 2)) orow_bf[col0 + j] = __float2bfloat16(v[j]);
      }
    }
    }
    if (p.push_out && (c & 3) == 3) {
      // drain one half of the width: the warp sends its 32 rows, two per store instruction
      // (256 contiguous bytes each) to the rank that owns them, so the NVLink writes are
      // full-width instead of 16-byte fragments.  Only this warp touches the block.
      __syncwarp();
      const int half = c >> 2;
      const long long row0 = warp_row0;
      const int owner = (int)(row0 / p.rows_per_owner);
      __nv_bfloat16* obase = reinterpret_cast<__nv_bfloat16*>(p.out_ptrs[owner]) +
                             (long long)p.rank * p.out_slot_stride +
                             (row0 - (long long)owner * p.rows_per_owner) * p.ldo +
                             (long long)nb * CG_BN + half * 128;
      const int unit = lane & 15;
      const int colu = nb * CG_BN + half * 128 + unit * 8;
#pragma unroll 4
      for (int rr = lane >> 4; rr < 32; rr += 2) {
        if (row0 + rr < p.M && colu < p.N) {
          const uint32_t addr = out_stage + quad * 8192 + rr * 256 + (((uint32_t)unit ^ (uint32_t)(rr & 15)) * 16);
          uint4 o;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(o.x), "=r"(o.y), "=r"(o.z), "=r"(o.w) : "r"(addr) : "memory");
          if (DZ_STORE_OK(obase + (long long)rr * p.ldo + unit * 8, 16))
            *reinterpret_cast<uint4*>(obase + (long long)rr * p.ldo + unit * 8) = o;
        }
      }
      __syncwarp();
    }
  }
}

template <int CG_STAGES>
__global__ void __launch_bounds__(CG_THREADS, 1)
comm_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const CommGemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[CG_STAGES];
  __shared__ __align__(8) uint64_t bar_empty[CG_STAGES];
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile int s_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int num_tiles = p.num_m * p.num_n;
  const int num_kb = (p.K + CG_BK - 1) / CG_BK;
  // CTAs that also push take the last join_tiles tiles of the order, the others the rest
  const bool pusher = (int)blockIdx.x < p.n_push;
  // (join_tiles < 0: the pushing CTAs multiply nothing)
  const bool split = p.n_push > 0 && p.n_push < (int)gridDim.x && p.join_tiles != 0;
  const int reg_tiles = (split && p.join_tiles > 0) ? num_tiles - p.join_tiles : num_tiles;
  const int cta = !split ? (int)blockIdx.x : (pusher ? reg_tiles + (int)blockIdx.x : (int)blockIdx.x - p.n_push);
  const int n_cta = !split ? (int)gridDim.x : (pusher ? p.n_push : (int)gridDim.x - p.n_push);
  const int tile_end = (split && !pusher) ? reg_tiles : num_tiles;
  // the table of the push warps sits behind the operand ring (where a push epilogue stages its rows)
  uint8_t* table_smem = smem_raw + ((smem_base - smem_u32(smem_raw)) + CG_STAGES * CG_STAGE_BYTES);

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < CG_STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_acc_full[a]), 1);
      mbar_init(smem_u32(&bar_acc_empty[a]), 4);
    }
    fence_mbar_init();
    if (num_tiles > 0) {          // a push-only launch carries no tensor maps
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&s_tmem_base), CG_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;

  if (warp >= CG_GEMM_THREADS / 32) {
    // ------------------------------------------------------------ push warps
    if (pusher) cg_push_role(p, table_smem, (int)threadIdx.x - CG_GEMM_THREADS);
  } else if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t seen = 0;      // bit s set: source s is known to have arrived
      for (int tile = cta; tile < tile_end && ok; tile += n_cta) {
        int mb, nb;
        cg_tile_coords(tile, p, CG_BM, mb, nb);
        if (p.gather) {
          // every source rank that owns a row of this tile's gathered operand must have arrived
          long long r0 = p.gather == 1 ? (long long)mb * CG_BM : (long long)nb * CG_BN;
          long long r1 = p.gather == 1 ? min(r0 + CG_BM, (long long)p.M) : min(r0 + CG_BN, (long long)p.N);
          bool fenced = true;
          for (long long rr = r0; rr < r1 && ok;) {
            long long q = p.src_period ? rr % p.src_period : rr;
            int src = (int)(q / p.rows_per_src);
            if (src >= p.world) src = p.world - 1;
            const bool chunked = p.gather == 1 && p.chunk_tiles > 0;
            const int chunk = chunked ? (int)((q % p.rows_per_src) / CG_BM) / p.chunk_tiles : 0;
            if ((src != p.rank || p.wait_self) && (chunked || !(seen & (1u << src)))) {
              if (!cg_wait_flag(p.ready_flags + src * CG_MAXC + chunk, p.ready_epoch, &s_abort, p.err)) {
                ok = false;
                break;
              }
              if (!chunked) seen |= 1u << src;
              fenced = false;
            }
            rr += p.rows_per_src - (q % p.rows_per_src);      // first row of the next owner
          }
          if (!ok) break;
          // the rows were written by a peer's ordinary stores; order them before TMA reads
          if (!fenced) asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1, &s_abort, p.err, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          uint32_t full = smem_u32(&bar_full[stage]);
          uint32_t a_dst = smem_base + stage * CG_STAGE_BYTES;
          uint32_t b_dst = a_dst + CG_A_BYTES;
          mbar_arrive_expect_tx(full, CG_STAGE_BYTES);
          tma_load_2d(a_dst, &tmA, full, kb * CG_BK, mb * CG_BM);
          tma_load_2d(b_dst, &tmB, full, kb * CG_BK, nb * CG_BN);
          if (++stage == CG_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(CG_BM, CG_BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cta; tile < tile_end && ok; tile += n_cta) {
        if (!mbar_wait(smem_u32(&bar_acc_empty[acc]), acc_phase ^ 1, &s_abort, p.err,
                       ERR_WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * CG_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &s_abort, p.err, ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          uint32_t a_src = smem_base + stage * CG_STAGE_BYTES;
          uint32_t b_src = a_src + CG_A_BYTES;
          uint64_t a_desc = umma_desc_k_sw128(a_src);
          uint64_t b_desc = umma_desc_k_sw128(b_src);
#pragma unroll
          for (int k = 0; k < CG_BK / 16; ++k)
            umma_bf16_ss(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
          umma_commit(smem_u32(&bar_empty[stage]));
          if (++stage == CG_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(smem_u32(&bar_acc_full[acc]));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t out_stage = smem_base + CG_STAGES * CG_STAGE_BYTES;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = cta; tile < tile_end; tile += n_cta) {
      int mb, nb;
      cg_tile_coords(tile, p, CG_BM, mb, nb);
      if (!mbar_wait(smem_u32(&bar_acc_full[acc]), acc_phase, &s_abort, p.err, ERR_WAIT_TMEM_FULL))
        break;
      tc_fence_after();
      const long long row = (long long)mb * CG_BM + row_in_tile;
      const uint32_t t_row = tmem_base + acc * CG_BN + (static_cast<uint32_t>(quad * 32) << 16);
      cg_drain_tile(p, t_row, row, (long long)mb * CG_BM + quad * 32, nb, quad, lane, out_stage);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[acc]));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (p.push_out) __threadfence_system();     // this CTA's remote tile stores are ordered
  }

  // ---------------------------------------------------------------- tear-down
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) {
    // the last GEMM CTA of this rank announces completion to the peers
    __threadfence_system();
    unsigned int old = atomicAdd(p.counters + 1, 1u);
    if (old + 1u == p.gemm_target && !s_abort) {
      __threadfence_system();
      if (p.push_out)
        for (int d = 0; d < p.world; ++d) cg_st_release_sys(p.rs_flag_ptrs[d] + p.rank, p.rs_epoch);
      if (p.gather && p.ack_ptrs)
        for (int d = 0; d < p.world; ++d) cg_st_release_sys(p.ack_ptrs[d] + p.rank, p.ack_epoch);
    }
  }
  if (warp == 1) {
    __syncwarp();
    if (s_abort) {
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, CG_TMEM_COLS);
  }
}


// ------------------------------------------------------------------------------------------------
// Two-SM variant: a cluster of two CTAs computes one 256 x 256 output tile with
// tcgen05.mma.cta_group::2 (the tile engine of gemm2_sm100.cu: CTA r of the pair stages rows
// [128 r, 128 r + 128) of the A tile and of the W tile, the leader issues the MMAs, each CTA drains
// its own 128 accumulator rows), with the same communication roles as the one-SM kernel above: push
// warps in the pushing CTAs, per-source waits before the first load of gathered rows (each CTA for
// the rows it loads itself), the reduce-scatter epilogue, acks.  Row extents that change owner must
// be multiples of 256 (all-gather) / 128 (reduce-scatter); the host falls back to the one-SM kernel
// otherwise.  chunk_tiles counts 256-row tiles here.
constexpr int C2_BM = 256;
constexpr int C2_STAGES_PLAIN = 6;
constexpr int C2_STAGES_PUSH = 5;                    // one stage makes room for the row staging
constexpr int C2_A_BYTES = 128 * CG_BK * 2;
constexpr int C2_B_BYTES = 128 * CG_BK * 2;
constexpr int C2_STAGE_BYTES = C2_A_BYTES + C2_B_BYTES;
constexpr int C2_SMEM_PLAIN = C2_STAGES_PLAIN * C2_STAGE_BYTES + CG_TABLE_BYTES + 1024;
constexpr int C2_SMEM_PUSH = C2_STAGES_PUSH * C2_STAGE_BYTES + CG_OUT_STAGE_BYTES + 1024;

template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(CG_THREADS, 1)
comm_gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const CommGemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[STAGES];      // used in the leader only
  __shared__ __align__(8) uint64_t bar_empty[STAGES];     // one per CTA
  __shared__ __align__(8) uint64_t bar_acc_full[2];       // one per CTA
  __shared__ __align__(8) uint64_t bar_acc_empty[2];      // used in the leader only
  __shared__ uint32_t s_tmem_base;
  __shared__ volatile int s_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();
  const bool leader = crank == 0;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int num_tiles = p.num_m * p.num_n;
  const int num_kb = (p.K + CG_BK - 1) / CG_BK;
  // tile shares in units of clusters (n_push is even: both CTAs of a pair push or neither does)
  const int cluster_id = (int)blockIdx.x >> 1;
  const int num_clusters = (int)gridDim.x >> 1;
  const int push_clusters = p.n_push >> 1;
  const bool pusher = (int)blockIdx.x < p.n_push;
  const bool split = push_clusters > 0 && push_clusters < num_clusters && p.join_tiles != 0;
  const int reg_tiles = (split && p.join_tiles > 0) ? num_tiles - p.join_tiles : num_tiles;
  const int cta = !split ? cluster_id : (pusher ? reg_tiles + cluster_id : cluster_id - push_clusters);
  const int n_cta = !split ? num_clusters : (pusher ? push_clusters : num_clusters - push_clusters);
  const int tile_end = (split && !pusher) ? reg_tiles : num_tiles;
  uint8_t* table_smem = smem_raw + ((smem_base - smem_u32(smem_raw)) + STAGES * C2_STAGE_BYTES);

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_acc_full[a]), 1);
      mbar_init(smem_u32(&bar_acc_empty[a]), 8);      // 4 epilogue warps x 2 CTAs
    }
    fence_mbar_init();
    if (num_tiles > 0) {
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
    }
  }
  if (warp == 1) {
    tmem_alloc_2sm(smem_u32(&s_tmem_base), CG_TMEM_COLS);
    tmem_relinquish_2sm();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;

  if (warp >= CG_GEMM_THREADS / 32) {
    // ------------------------------------------------------------ push warps
    if (pusher) cg_push_role(p, table_smem, (int)threadIdx.x - CG_GEMM_THREADS);
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (each CTA)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t seen = 0;
      for (int tile = cta; tile < tile_end && ok; tile += n_cta) {
        int mb, nb;
        cg_tile_coords(tile, p, C2_BM, mb, nb);
        if (p.gather) {
          // the source ranks that own the 128 gathered rows THIS CTA loads must have arrived
          long long r0 = (p.gather == 1 ? (long long)mb * C2_BM : (long long)nb * CG_BN) + (long long)crank * 128;
          long long r1 = min(r0 + 128, (long long)(p.gather == 1 ? p.M : p.N));
          bool fenced = true;
          for (long long rr = r0; rr < r1 && ok;) {
            long long q = p.src_period ? rr % p.src_period : rr;
            int src = (int)(q / p.rows_per_src);
            if (src >= p.world) src = p.world - 1;
            const bool chunked = p.gather == 1 && p.chunk_tiles > 0;
            const int chunk = chunked ? (int)((q % p.rows_per_src) / C2_BM) / p.chunk_tiles : 0;
            if ((src != p.rank || p.wait_self) && (chunked || !(seen & (1u << src)))) {
              if (!cg_wait_flag(p.ready_flags + src * CG_MAXC + chunk, p.ready_epoch, &s_abort, p.err)) {
                ok = false;
                break;
              }
              if (!chunked) seen |= 1u << src;
              fenced = false;
            }
            rr += p.rows_per_src - (q % p.rows_per_src);
          }
          if (!ok) break;
          if (!fenced) asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1, &s_abort, p.err, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t full_local = smem_u32(&bar_full[stage]);
          const uint32_t full_leader = map_to_cta(full_local, 0);
          const uint32_t a_dst = smem_base + stage * C2_STAGE_BYTES;
          const uint32_t b_dst = a_dst + C2_A_BYTES;
          if (leader) mbar_arrive_expect_tx(full_local, 2 * C2_STAGE_BYTES);   // both CTAs' bytes
          tma_load_2d_2sm(a_dst, &tmA, full_leader, kb * CG_BK, mb * C2_BM + (int)crank * 128);
          tma_load_2d_2sm(b_dst, &tmB, full_leader, kb * CG_BK, nb * CG_BN + (int)crank * 128);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA)
    if (leader && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(C2_BM, CG_BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cta; tile < tile_end && ok; tile += n_cta) {
        if (!mbar_wait_cluster(smem_u32(&bar_acc_empty[acc]), acc_phase ^ 1, &s_abort, p.err,
                               ERR_WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * CG_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &s_abort, p.err, ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_src = smem_base + stage * C2_STAGE_BYTES;
          const uint32_t b_src = a_src + C2_A_BYTES;
          const uint64_t a_desc = umma_desc_k_sw128(a_src);
          const uint64_t b_desc = umma_desc_k_sw128(b_src);
#pragma unroll
          for (int k = 0; k < CG_BK / 16; ++k)
            umma_bf16_ss_2sm(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
          umma_commit_2sm(smem_u32(&bar_empty[stage]), 3);      // frees the stage in both CTAs
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_2sm(smem_u32(&bar_acc_full[acc]), 3);       // wakes both epilogues
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (each CTA: its 128 rows)
    const int quad = warp & 3;
    const uint32_t out_stage = smem_base + STAGES * C2_STAGE_BYTES;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = cta; tile < tile_end; tile += n_cta) {
      int mb, nb;
      cg_tile_coords(tile, p, C2_BM, mb, nb);
      if (!mbar_wait(smem_u32(&bar_acc_full[acc]), acc_phase, &s_abort, p.err, ERR_WAIT_TMEM_FULL))
        break;
      tc_fence_after();
      const long long warp_row0 = (long long)mb * C2_BM + (long long)crank * 128 + quad * 32;
      const uint32_t t_row = tmem_base + acc * CG_BN + (static_cast<uint32_t>(quad * 32) << 16);
      cg_drain_tile(p, t_row, warp_row0 + lane, warp_row0, nb, quad, lane, out_stage);
      // this CTA's half of the accumulator is drained: tell the leader's MMA issuer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bar_acc_empty[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (p.push_out) __threadfence_system();
  }

  // ---------------------------------------------------------------- tear-down
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    unsigned int old = atomicAdd(p.counters + 1, 1u);
    if (old + 1u == p.gemm_target && !s_abort) {
      __threadfence_system();
      if (p.push_out)
        for (int d = 0; d < p.world; ++d) cg_st_release_sys(p.rs_flag_ptrs[d] + p.rank, p.rs_epoch);
      if (p.gather && p.ack_ptrs)
        for (int d = 0; d < p.world; ++d) cg_st_release_sys(p.ack_ptrs[d] + p.rank, p.ack_epoch);
    }
    if (s_abort) {
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
  }
  cluster_sync_all();          // neither CTA leaves while the other may still read its shared memory
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, CG_TMEM_COLS);
  }
}

}  // namespace dz

using namespace dz;
DZ_DEBUG_TU(commgemm)

// Plain-C mirror of the launch description (filled by Python through ctypes).
struct DzCommGemmDesc {
  // GEMM
  const void* A; long long lda; const void* W; long long ldw;
  void* out; long long ldo; const void* bias; const void* residual; long long ldr;
  int M, N, K, act, out_fp32; float out_scale;
  // gather
  int gather, rows_per_src, src_period, wait_self; const void* ready_flags; unsigned int ready_epoch;
  const void* ack_ptrs; unsigned int ack_epoch;
  // push epilogue
  int push_out; const void* out_ptrs; long long out_slot_stride; int rows_per_owner;
  const void* rs_flag_ptrs; unsigned int rs_epoch;
  // push role
  int n_push, push_nseg; const void* push_src[3]; long long push_ld, push_rows, push_cols;
  const void* push_dst_ptrs; long long push_dst_ld, push_dst_row0[3]; int push_to_self;
  const void* push_flag_ptrs; unsigned int push_epoch;
  const void* push_wait_acks; unsigned int push_wait_epoch;
  int push_perturb; unsigned long long push_seed; float push_coef; int push_tensor_id[3];
  long long push_elem_base[3]; const void* gauss_table;
  // bookkeeping
  int rank, world; void* counters; unsigned int push_target, gemm_target;
  int two_sm;                    // 1: run the two-SM kernel (the caller asked dz_comm_gemm_two_sm first)
  int chunk_rows;                // all-gather -> GEMM: rows per progress chunk of a source (0 = one chunk)
  int join_tiles;                // tiles at the end of the order left to the pushing CTAs (0 = no split)
};

extern "C" int dz_comm_gemm_desc_bytes() { return (int)sizeof(DzCommGemmDesc); }

// Whether a launch of this shape runs the two-SM kernel: enough 256 x 256 tiles for one wave of CTA pairs,
// and - when rows of A arrive from peers - ownership and progress chunks in whole 256-row tiles.
extern "C" int dz_comm_gemm_two_sm(int M, int N, int gather, int rows_per_src, int chunk_rows) {
  if (M <= 0 || N <= 0) return 0;
  const long long tiles = (long long)((M + C2_BM - 1) / C2_BM) * ((N + CG_BN - 1) / CG_BN);
  if (tiles < sm_count() / 2) return 0;
  if (gather == 1 && ((rows_per_src % C2_BM) || (chunk_rows % C2_BM))) return 0;
  return 1;
}
extern "C" int dz_comm_gemm_tiles(int M, int N, int two_sm) {
  const int bm = two_sm ? C2_BM : CG_BM;
  return ((M + bm - 1) / bm) * ((N + CG_BN - 1) / CG_BN);
}
// CTAs of a launch of this shape with n_push pushing CTAs: one per output tile (two per 256 x 256 tile of the
// two-SM kernel) up to the SM count, and at least the pushing ones.  The host keeps its completion counters
// in step with it.
extern "C" int dz_comm_gemm_grid(int M, int N, int n_push, int two_sm) {
  const int sms = sm_count() & ~1;
  const long long tiles = (M > 0 && N > 0) ? dz_comm_gemm_tiles(M, N, two_sm) : 0;
  long long g = two_sm ? 2 * tiles : tiles;
  if (g > sms) g = sms;
  if (n_push > g) g = n_push < sms ? n_push : sms;
  if (two_sm) g = (g + 1) & ~1ll;
  return (int)g;
}

extern "C" int dz_comm_gemm(const DzCommGemmDesc* d, uint32_t* err, cudaStream_t stream) {
  if (!d) return DZ_ERR_ARG;
  const bool has_gemm = d->M > 0 && d->N > 0 && d->K > 0;
  const bool two = has_gemm && d->two_sm &&
                   dz_comm_gemm_two_sm(d->M, d->N, d->gather, d->rows_per_src, d->chunk_rows);
  if (d->two_sm && !two) return DZ_ERR_ARG;
  const int BM = two ? C2_BM : CG_BM;
  if (!has_gemm && d->n_push <= 0) return DZ_ERR_ARG;
  if (d->world <= 0 || d->world > CG_MAX_WORLD || d->rank < 0 || d->rank >= d->world) return DZ_ERR_ARG;
  CommGemmArgs a{};
  CUtensorMap tmA{}, tmB{};
  if (has_gemm) {
    if (!d->A || !d->W) return DZ_ERR_ARG;
    if ((d->K & 7) || (d->lda & 7) || (d->ldw & 7) || (d->ldo & 7)) return DZ_ERR_ALIGN;
    if (d->gather && (d->rows_per_src <= 0 || !d->ready_flags)) return DZ_ERR_ARG;
    if (d->gather == 1 && (d->rows_per_src % (two ? C2_BM : CG_BM))) return DZ_ERR_ALIGN;
    if (d->push_out && (!d->out_ptrs || !d->rs_flag_ptrs || d->rows_per_owner <= 0 ||
                        (d->rows_per_owner % CG_BM) || d->out_fp32))
      return DZ_ERR_ARG;
    if (!d->push_out && !d->out) return DZ_ERR_ARG;
    if (d->push_out && (d->N & 7)) return DZ_ERR_ALIGN;
    int rc = make_tmap_bf16_2d(&tmA, d->A, d->M, d->K, d->lda, 128, CG_BK, true);
    if (rc) return rc;
    rc = make_tmap_bf16_2d(&tmB, d->W, d->N, d->K, d->ldw, two ? 128 : CG_BN, CG_BK, true);
    if (rc) return rc;
    a.M = d->M; a.N = d->N; a.K = d->K;
    a.num_m = (d->M + BM - 1) / BM;
    a.num_n = (d->N + CG_BN - 1) / CG_BN;
  }
  if (d->n_push > 0) {
    if (d->push_nseg < 1 || d->push_nseg > 3 || !d->push_dst_ptrs || !d->push_flag_ptrs ||
        (d->push_cols & 7) || (d->push_ld & 7) || (d->push_dst_ld & 7))
      return DZ_ERR_ARG;
    for (int sgi = 0; sgi < d->push_nseg; ++sgi) {
      if (!d->push_src[sgi]) return DZ_ERR_ARG;
      if (d->push_perturb && (d->push_elem_base[sgi] & 7)) return DZ_ERR_ARG;
    }
    if (d->push_perturb && (!d->gauss_table || d->push_out)) return DZ_ERR_ARG;
  }
  a.out = d->out; a.ldo = d->ldo;
  a.bias = (const __nv_bfloat16*)d->bias; a.residual = (const __nv_bfloat16*)d->residual; a.ldr = d->ldr;
  a.act = d->act; a.out_fp32 = d->out_fp32; a.out_scale = d->out_scale;
  a.wide_store = d->out && !d->out_fp32 && !(reinterpret_cast<uintptr_t>(d->out) & 31) && !(d->ldo & 15);
  a.gather = has_gemm ? d->gather : 0; a.rows_per_src = d->rows_per_src; a.wait_self = d->wait_self;
  a.src_period = d->src_period;
  a.ready_flags = (const uint32_t*)d->ready_flags; a.ready_epoch = d->ready_epoch;
  a.ack_ptrs = (uint32_t* const*)d->ack_ptrs; a.ack_epoch = d->ack_epoch;
  a.push_out = d->push_out; a.out_ptrs = (void* const*)d->out_ptrs;
  a.out_slot_stride = d->out_slot_stride; a.rows_per_owner = d->rows_per_owner;
  a.rs_flag_ptrs = (uint32_t* const*)d->rs_flag_ptrs; a.rs_epoch = d->rs_epoch;
  a.n_push = d->n_push > 0 ? d->n_push : 0;
  if (a.n_push > sm_count()) a.n_push = sm_count();
  a.push_nseg = d->push_nseg;
  for (int sgi = 0; sgi < 3; ++sgi) {
    a.push_src[sgi] = (const __nv_bfloat16*)d->push_src[sgi];
    a.push_dst_row0[sgi] = d->push_dst_row0[sgi];
    a.push_tensor_id[sgi] = d->push_tensor_id[sgi];
    a.push_elem_base[sgi] = d->push_elem_base[sgi];
  }
  a.push_ld = d->push_ld;
  a.push_rows = d->push_rows; a.push_cols = d->push_cols;
  a.push_dst_ptrs = (void* const*)d->push_dst_ptrs; a.push_dst_ld = d->push_dst_ld;
  a.push_to_self = d->push_to_self;
  if (d->chunk_rows > 0) {
    // chunks are whole row tiles, at most CG_MAXC of them per source
    if (d->chunk_rows % BM || d->push_perturb) return DZ_ERR_ARG;
    if (d->n_push > 0 && (d->push_rows + d->chunk_rows - 1) / d->chunk_rows > CG_MAXC) return DZ_ERR_ARG;
    if (has_gemm && d->gather == 1 &&
        (d->rows_per_src % d->chunk_rows || d->rows_per_src / d->chunk_rows > CG_MAXC))
      return DZ_ERR_ARG;
    a.push_chunk_rows = d->chunk_rows;
    a.chunk_tiles = d->chunk_rows / BM;
  }
  a.push_flag_ptrs = (uint32_t* const*)d->push_flag_ptrs; a.push_epoch = d->push_epoch;
  a.push_wait_acks = (const uint32_t*)d->push_wait_acks; a.push_wait_epoch = d->push_wait_epoch;
  a.push_perturb = d->push_perturb; a.push_seed = d->push_seed; a.push_coef = d->push_coef;
  a.gauss_table = (const uint32_t*)d->gauss_table;
  a.rank = d->rank; a.world = d->world; a.counters = (unsigned int*)d->counters;
  a.push_target = d->push_target; a.gemm_target = d->gemm_target; a.err = err;
  if (!a.counters) return DZ_ERR_ARG;
  static PerDeviceFlag configured, configured2p, configured2;
  if (int rc_cfg = ensure_dyn_smem(configured, comm_gemm_kernel<CG_STAGES_PUSH>, CG_SMEM_PUSH)) return rc_cfg;
  if (int rc_cfg = ensure_dyn_smem(configured2p, comm_gemm2_kernel<C2_STAGES_PUSH>, C2_SMEM_PUSH)) return rc_cfg;
  if (int rc_cfg = ensure_dyn_smem(configured2, comm_gemm2_kernel<C2_STAGES_PLAIN>, C2_SMEM_PLAIN)) return rc_cfg;
  if (two) a.n_push = (a.n_push + 1) & ~1;          // both CTAs of a pair push, or neither
  // one CTA per SM at most: every CTA must be resident at once (the roles wait on one another through flags)
  const int grid = dz_comm_gemm_grid(has_gemm ? d->M : 0, has_gemm ? d->N : 0, a.n_push, two);
  if (grid < 1 || grid > sm_count() || a.n_push > grid) return DZ_ERR_TOO_LARGE;
  if (has_gemm && a.n_push > 0 && a.n_push < grid && d->join_tiles != 0) {
    // join_tiles 0: every CTA strides over all tiles; > 0: the pushing CTAs take that many tiles at the end of
    // the order; < 0: the pushing CTAs multiply nothing
    if (d->join_tiles >= a.num_m * a.num_n) return DZ_ERR_ARG;
    a.join_tiles = d->join_tiles;
  }
  if (two && a.push_out)
    comm_gemm2_kernel<C2_STAGES_PUSH><<<grid, CG_THREADS, C2_SMEM_PUSH, stream>>>(tmA, tmB, a);
  else if (two)
    comm_gemm2_kernel<C2_STAGES_PLAIN><<<grid, CG_THREADS, C2_SMEM_PLAIN, stream>>>(tmA, tmB, a);
  else if (a.push_out)
    comm_gemm_kernel<CG_STAGES_PUSH><<<grid, CG_THREADS, CG_SMEM_PUSH, stream>>>(tmA, tmB, a);
  else
    comm_gemm_kernel<CG_STAGES_PLAIN><<<grid, CG_THREADS, CG_SMEM_PLAIN, stream>>>(tmA, tmB, a);
  return cuda_rc(cudaGetLastError());
}
