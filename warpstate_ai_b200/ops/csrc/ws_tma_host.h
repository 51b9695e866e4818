// Host-side creation of TMA tensor maps (driver entry point resolved at run time, so the
// library does not link against libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <mutex>
#include <stdint.h>
#include <stdio.h>

namespace ws {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is a driver call and wants a context current on the calling thread; the
// runtime binds the primary context lazily, on a thread's first runtime call that needs one.  A thread
// whose first CUDA action is building a tensor map (an autograd worker whose tensors all came out of
// the caching allocator) otherwise gets CUDA_ERROR_INVALID_CONTEXT.  Once per thread.
inline void ensure_context_on_this_thread() {
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

inline EncodeTiledFn get_encode_fn() {
  ensure_context_on_this_thread();
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// 2-D BF16 tensor map with 128-byte swizzle: `inner` contiguous elements per row, `outer` rows,
// row pitch `ld` elements, box = box_inner x box_outer (box_inner * 2 bytes <= 128).
inline int make_map_bf16_swz(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                             uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle);

inline int make_map_bf16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer,
                         uint64_t ld, uint32_t box_inner, uint32_t box_outer) {
  return make_map_bf16_swz(map, base, inner, outer, ld, box_inner, box_outer, CU_TENSOR_MAP_SWIZZLE_128B);
}

// The same with a chosen swizzle (box_inner * 2 bytes must not exceed the swizzle span).
inline int make_map_bf16_swz(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                             uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -10;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * 2) % 16 != 0) return -11;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)  // say what was refused: the bare code cannot be traced back to an operand
    fprintf(stderr, "ws_b200: tensor-map encode refused (CUresult %d): map %p base %p dims %llu x %llu pitch %llu B box %u x %u swizzle %d\n",
            (int)r, (void*)map, base, (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)(ld * 2),
            box_inner, box_outer, (int)swizzle);
  return r == CUDA_SUCCESS ? 0 : -12;
}

// 2-D FP32 tensor map (128-byte swizzle): for the shared-memory-staged FP32 epilogues.
inline int make_map_f32(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                        uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -10;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * 4) % 16 != 0) return -11;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 4};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}

}  // namespace ws
