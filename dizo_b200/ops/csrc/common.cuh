// Shared device helpers for the sm_100a kernels: PTX wrappers for mbarrier, TMA
// (cp.async.bulk.tensor), tcgen05 (TMEM alloc / MMA / commit / ld), bounded waits
// and the error word protocol.
//
// Error word protocol: every kernel that can wait on something receives a pointer
// to a 32-bit word in global memory.  A wait that exceeds its time limit stores a
// non-zero code there (first writer wins), raises a CTA-local abort flag, and every
// role of the CTA falls through to the common tear-down (TMEM is released, the
// kernel returns).  The host reads the word after synchronising.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace dz {

// ---------------------------------------------------------------- error codes
enum : uint32_t {
  ERR_NONE = 0,
  ERR_WAIT_FULL = 1,       // consumer waited for a TMA-filled stage
  ERR_WAIT_EMPTY = 2,      // producer waited for a free stage
  ERR_WAIT_TMEM_FULL = 3,  // epilogue waited for an accumulator
  ERR_WAIT_TMEM_EMPTY = 4, // MMA issuer waited for a drained accumulator
  ERR_WAIT_PEER = 5,       // wait on a flag written by another GPU
  ERR_WAIT_MISC = 6,
  ERR_BAD_ARG = 7,
};

#ifndef DZ_WAIT_TIMEOUT_NS
#define DZ_WAIT_TIMEOUT_NS 2000000000ull  // 2 s per wait, then the kernel gives up
#endif

// ---------------------------------------------------------------- debug build: checked stores
// Compiled with -DDZ_DEBUG_BOUNDS (python -m dizo_b200.ops.build --debug-bounds) every global store of
// the kernels first checks that its bytes fall inside one of the address ranges the host registered
// for the launch (the tensors handed to the entry points and the peers' symmetric regions).  A store
// outside every range is SKIPPED, counted, and its address and source line kept; nothing traps and the
// context stays usable.  The host reads the record back after synchronising (ops/_lib.py).  This stands
// in for compute-sanitizer's memcheck on boxes where that tool is closed.  One state per translation
// unit (no relocatable device code needed); DZ_DEBUG_TU(name) exports its set / get entry points.
#ifdef DZ_DEBUG_BOUNDS
constexpr int DZ_DBG_MAX_RANGES = 256;
struct DzDebugState {
  unsigned long long lo[DZ_DBG_MAX_RANGES], hi[DZ_DBG_MAX_RANGES];
  int n;                         // 0 = not armed: every store passes
  unsigned int violations;
  unsigned long long first_addr;
  int first_line;
  int pad;
};
static __device__ DzDebugState g_dz_dbg;
__device__ __forceinline__ bool dz_store_ok(const void* p, unsigned long long bytes, int line) {
  const int n = g_dz_dbg.n;
  if (n == 0) return true;
  const unsigned long long a = reinterpret_cast<unsigned long long>(p);
  for (int i = 0; i < n; ++i)
    if (a >= g_dz_dbg.lo[i] && a + bytes <= g_dz_dbg.hi[i]) return true;
  if (atomicAdd(&g_dz_dbg.violations, 1u) == 0u) {
    g_dz_dbg.first_addr = a;
    g_dz_dbg.first_line = line;
  }
  return false;
}
#define DZ_STORE_OK(p, bytes) (dz::dz_store_ok((p), (bytes), __LINE__))
#define DZ_DEBUG_TU(name)                                                                              \
  extern "C" int dz_debug_set_##name(const void* host_state) {                                         \
    return (int)cudaMemcpyToSymbol(dz::g_dz_dbg, host_state, sizeof(dz::DzDebugState));                \
  }                                                                                                    \
  extern "C" int dz_debug_get_##name(void* host_state) {                                               \
    return (int)cudaMemcpyFromSymbol(host_state, dz::g_dz_dbg, sizeof(dz::DzDebugState));              \
  }
#else
#define DZ_STORE_OK(p, bytes) (true)
#define DZ_DEBUG_TU(name)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "elect.sync _|P1, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P1;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P1;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when the CTA is aborting (this wait or another one
// ran out of time); the caller must leave its loop and go to the tear-down.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t* err_word, uint32_t code) {
  if (mbar_try_wait(bar, parity)) return true;
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      uint64_t now = global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > DZ_WAIT_TIMEOUT_NS) {
        *abort_flag = 1;
        if (err_word) atomicCAS(err_word, 0u, code | (blockIdx.x << 8));
        return false;
      }
    }
  }
  return true;
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load global -> this CTA's shared memory, completion on an mbarrier.
// No cluster multicast is ever used.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x,
                                            int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; bf16 inputs, fp32 accumulate.  One thread issues.
__device__ __forceinline__ void umma_bf16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same with the A operand in TMEM (bf16 pairs packed in 32-bit columns, one row per lane).
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier of this CTA once all previously issued MMAs have finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane
// (base_lane + i), registers r[0..31] = columns col .. col+31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Thread i of the warp writes r[0..15] to lane (base_lane + i), columns col .. col+15.
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
      "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
      "r"(r[15])
      : "memory");
}

// Shared-memory matrix descriptor for a bf16 tile stored K-major with the 128-byte
// swizzle (the layout a TMA load with CU_TENSOR_MAP_SWIZZLE_128B and a 64-element
// inner box produces): rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);        // start address
  d |= static_cast<uint64_t>(1) << 16;                           // leading byte offset (unused here)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                   // stride byte offset: 8 rows
  d |= static_cast<uint64_t>(1) << 46;                           // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                           // SWIZZLE_128B
  return d;
}
// MN-major variant (the contiguous direction of the tile in shared memory is M/N,
// 64 elements = 128 bytes per swizzle row, 8 K-rows per 1024-byte group).
// lbo_bytes: distance between consecutive 64-element blocks along M/N;
// sbo_bytes: distance between consecutive groups of 8 along K.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                       uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32, dense.  a_mn / b_mn = 1 when the
// operand is MN-major in shared memory.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N, int a_mn = 0, int b_mn = 0) {
  return (1u << 4)                       // accumulator fp32
         | (1u << 7)                     // A bf16
         | (1u << 10)                    // B bf16
         | (static_cast<uint32_t>(a_mn) << 15) | (static_cast<uint32_t>(b_mn) << 16) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// ---------------------------------------------------------------- small math
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// 32 consecutive bf16 outputs of one lane's row: two 32-byte stores (one whole sector each) when the address allows,
// else four 16-byte stores.
__device__ __forceinline__ void store_row32(__nv_bfloat16* op, const uint4 (&o)[4], bool wide) {
  if (wide) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (DZ_STORE_OK(op + h * 16, 32))
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(op + h * 16),
                     "r"(o[2 * h].x), "r"(o[2 * h].y), "r"(o[2 * h].z), "r"(o[2 * h].w), "r"(o[2 * h + 1].x),
                     "r"(o[2 * h + 1].y), "r"(o[2 * h + 1].z), "r"(o[2 * h + 1].w)
                     : "memory");
    }
  } else {
    uint4* op4 = reinterpret_cast<uint4*>(op);
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (DZ_STORE_OK(op4 + q, 16)) op4[q] = o[q];
  }
}

__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
}

}  // namespace dz
