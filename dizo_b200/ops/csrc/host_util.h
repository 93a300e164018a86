// Host-side helpers shared by the launchers: TMA descriptor encoding through the
// driver entry point (no link-time dependency on libcuda), argument checks.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace dz {

// Return codes of the extern "C" entry points (0 = success; CUDA errors are returned
// as 1000 + cudaError_t).
enum : int {
  DZ_OK = 0,
  DZ_ERR_ARG = 1,
  DZ_ERR_ALIGN = 2,
  DZ_ERR_TMAP = 3,
  DZ_ERR_TOO_LARGE = 4,
  DZ_ERR_CUDA_BASE = 1000,
};

inline int cuda_rc(cudaError_t e) { return e == cudaSuccess ? DZ_OK : DZ_ERR_CUDA_BASE + (int)e; }

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !p) return nullptr;
    fn = reinterpret_cast<PFN_encodeTiled>(p);
  }
  return fn;
}

// 2-D bf16 tensor [rows, cols] with row stride ld (elements); box = [box_rows, box_cols];
// 128-byte swizzle (box_cols * 2 bytes must equal 128) or none.
inline int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                             uint64_t ld, uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return DZ_ERR_TMAP;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return DZ_ERR_ALIGN;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DZ_OK : DZ_ERR_TMAP;
}

// 3-D bf16 tensor [d2, d1, d0] (d0 innermost) with strides in elements.
inline int make_tmap_bf16_3d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1,
                             uint64_t d2, uint64_t stride1, uint64_t stride2, uint32_t box0,
                             uint32_t box1, uint32_t box2, bool swizzle128) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return DZ_ERR_TMAP;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((stride1 * 2) & 15) || ((stride2 * 2) & 15))
    return DZ_ERR_ALIGN;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1 * 2, stride2 * 2};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DZ_OK : DZ_ERR_TMAP;
}

// Launch attributes and device properties are per device, and one process may drive several GPUs:
// both are cached per device index, not per process.
constexpr int DZ_MAX_DEVICES = 64;

inline int sm_count() {
  static int n[DZ_MAX_DEVICES] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const bool cached = dev >= 0 && dev < DZ_MAX_DEVICES;
  if (cached && n[dev]) return n[dev];
  int v = 0;
  cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
  if (v <= 0) v = 148;
  if (cached) n[dev] = v;
  return v;
}

struct PerDeviceFlag {
  bool set[DZ_MAX_DEVICES] = {};
};

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device).
template <class Kern>
inline int ensure_dyn_smem(PerDeviceFlag& f, Kern kern, int bytes) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_rc(e);
  const bool cached = dev >= 0 && dev < DZ_MAX_DEVICES;
  if (cached && f.set[dev]) return DZ_OK;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return cuda_rc(e);
  if (cached) f.set[dev] = true;
  return DZ_OK;
}

}  // namespace dz
