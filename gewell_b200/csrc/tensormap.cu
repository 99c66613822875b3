// Host-side TMA descriptor encoding.  cuTensorMapEncodeTiled is a driver API
// entry point; it is looked up through the runtime so that the library links
// against the CUDA runtime only.
#include <cudaTypedefs.h>

#include <mutex>
#include <string>

#include "common.cuh"
#include "gemm_tc.cuh"

namespace gw {
namespace {

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(entry);
  });
  return fn;
}

}  // namespace

bool encode_tensor_map_2d(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows,
                          uint32_t box_rows, std::string* error, uint64_t pitch_bytes) {
  if (pitch_bytes == 0) pitch_bytes = row_bytes;
  auto fn = encode_fn();
  if (fn == nullptr) {
    if (error) *error = "cuTensorMapEncodeTiled is not available from this driver";
    return false;
  }
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || row_bytes % 16 != 0 || pitch_bytes % 16 != 0 ||
      pitch_bytes < row_bytes || rows == 0 || box_rows == 0 || box_rows > 256) {
    if (error) *error = "tensor map needs a 16-byte aligned base, a row pitch divisible by 16 and 1..256 box rows";
    return false;
  }
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t element_strides[2] = {1, 1};
  const CUresult status = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                             element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (status != CUDA_SUCCESS) {
    if (error) *error = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(int(status));
    return false;
  }
  return true;
}

bool encode_tensor_map_scales(CUtensorMap* map, const void* base, uint64_t k_atoms, uint64_t row_blocks,
                              uint32_t box_row_blocks, std::string* error) {
  auto fn = encode_fn();
  if (fn == nullptr) {
    if (error) *error = "cuTensorMapEncodeTiled is not available from this driver";
    return false;
  }
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || k_atoms == 0 || row_blocks == 0 || box_row_blocks == 0) {
    if (error) *error = "scale tensor map needs a 16-byte aligned base and positive extents";
    return false;
  }
  const cuuint64_t dims[2] = {k_atoms * 64, row_blocks};          // 8-byte words per row block, row blocks
  const cuuint64_t strides[1] = {k_atoms * 512};
  const cuuint32_t box[2] = {256, box_row_blocks};                // 4 atoms of 512 bytes
  const cuuint32_t element_strides[2] = {1, 1};
  const CUresult status = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(base), dims, strides, box,
                             element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (status != CUDA_SUCCESS) {
    if (error) *error = "cuTensorMapEncodeTiled (scales) failed with CUresult " + std::to_string(int(status));
    return false;
  }
  return true;
}

}  // namespace gw
