// Host side of the TMA tile loads: tensor maps for (B, S, H, D) tensors of 16-bit elements whose tiles are 128
// consecutive rows of one (batch, head) - the K/V tiles of the dense attention mode and the key tiles of the
// group-mass kernel.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <cstring>

#include "kernels.cuh"

namespace mcs {

namespace {

// cuTensorMapEncodeTiled through the runtime's driver entry point query (no link-time dependency on the driver)
PFN_cuTensorMapEncodeTiled tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled>(f);
  }();
  return fn;
}

}  // namespace

// 4-D tensor map of a (B, S, H, D) tensor of 16-bit elements with element strides {batch, row, head}: D innermost,
// then head / row / batch in the order of ascending stride (dimensions of extent 1 last, packed).  Box: 64
// elements (128 bytes, the swizzle span) x 128 rows.  Returns false if the layout cannot be described.
bool encode_tile_map(const void* base, const int64_t* stride, int B, int S, int H, int D, unsigned long long* out,
                     int& pos_h, int& pos_row, int& pos_b) {
  PFN_cuTensorMapEncodeTiled enc = tensor_map_encoder();
  if (enc == nullptr) return false;
  struct Dim { int which; unsigned long long extent; long long stride_bytes; };
  Dim d[3] = {{0, (unsigned long long)H, 2 * stride[2]}, {1, (unsigned long long)S, 2 * stride[1]}, {2, (unsigned long long)B, 2 * stride[0]}};
  std::stable_sort(d, d + 3, [](const Dim& a, const Dim& b) {
    const bool a1 = a.extent == 1, b1 = b.extent == 1;
    if (a1 != b1) return b1;                     // extent-1 dimensions go last
    return a.stride_bytes < b.stride_bytes;
  });
  unsigned long long prev_end = (unsigned long long)D * 2;
  cuuint64_t dims[4] = {(cuuint64_t)D, 0, 0, 0};
  cuuint64_t strides[3];
  cuuint32_t box[4] = {64, 1, 1, 1}, estr[4] = {1, 1, 1, 1};
  for (int i = 0; i < 3; ++i) {
    long long sb = d[i].stride_bytes;
    if (d[i].extent == 1) sb = (long long)prev_end;           // any valid stride: the coordinate is always 0
    if (sb <= 0 || (sb % 16) != 0 || (unsigned long long)sb < prev_end) return false;   // overlapping or misaligned
    dims[i + 1] = d[i].extent;
    strides[i] = (cuuint64_t)sb;
    prev_end = (unsigned long long)sb * d[i].extent;
    if (d[i].which == 0) pos_h = i + 1;
    if (d[i].which == 1) { pos_row = i + 1; box[i + 1] = 128; }
    if (d[i].which == 2) pos_b = i + 1;
  }
  CUtensorMap tm;
  const CUresult r = enc(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
  memcpy(out, &tm, 128);
  return true;
}

}  // namespace mcs
