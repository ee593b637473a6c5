// Host helpers: TMA tensor-map encoding through the driver entry point (no link-time
// dependency on libcuda, so the library builds on machines without a GPU driver).
#include "common.cuh"

#include <cudaTypedefs.h>
#include <mutex>

namespace trlb_host {

static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_elems,
                      uint32_t box_rows, uint32_t box_cols) {
  auto fn = get_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((row_stride_elems * 2) & 15)) return -2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_elems,
                      uint64_t stride2_elems, uint32_t b0, uint32_t b1, uint32_t b2) {
  auto fn = get_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((stride1_elems * 2) & 15) || ((stride2_elems * 2) & 15)) return -2;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_elems * 2, stride2_elems * 2};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

static bool g_pdl = false;
bool pdl_enabled() { return g_pdl; }

}  // namespace trlb_host

// Switches programmatic dependent launch of the decode-path kernels on or off for this process; returns the
// previous setting.  Set it before a CUDA graph is captured: the choice is baked into the graph's edges.
TRLB_API int trlb_set_pdl(int on) {
  const bool was = trlb_host::g_pdl;
  trlb_host::g_pdl = on != 0;
  return was ? 1 : 0;
}

TRLB_API int trlb_sm_count() { return trlb_host::sm_count(); }
