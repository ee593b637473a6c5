// Mixture-of-experts glue kernels around the grouped GEMM: weighted combine of the per-expert outputs back into token
// order.  Gather based (every output row reads its k source rows), so there are no atomics and the result does not
// depend on scheduling.
#include "common.cuh"

namespace trlb {

// y [T*k, H] bf16 in expert-sorted order; inv [T, k]: row of y holding (token t, choice j); w [T, k] fp32 weights.
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ inv,
                                   const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int T, int k, int H) {
  const int t = blockIdx.x;
  if (t >= T) return;
  const int nvec = H >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const int row = inv[(size_t)t * k + j];
      const float wj = w[(size_t)t * k + j];
      const uint4 u = reinterpret_cast<const uint4*>(y + (size_t)row * H)[v];
      const uint32_t q[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack_bf16(q[i]);
        acc[2 * i] = fmaf(wj, f.x, acc[2 * i]);
        acc[2 * i + 1] = fmaf(wj, f.y, acc[2 * i + 1]);
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]);
    o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]);
    o.w = pack_bf16(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + (size_t)t * H)[v] = o;
  }
}

// Expert-parallel dispatch by pulling: segment g = rows [src_row[g], src_row[g] + rows[g]) of rank src[g]'s buffer go to
// rows [dst_row[g], ...) of the local buffer.  One row (H bf16) per CTA iteration, 16 bytes per thread, so a full grid
// keeps a few MB in flight, which is what the NVLink round trip needs.  Each remote row crosses the link once; the
// grouped GEMM then reads the local copy as often as it has N tiles.
struct PullParams {
  const __nv_bfloat16* src[8];
};

__global__ void __launch_bounds__(256)
moe_pull_rows_kernel(const PullParams pp, const int* __restrict__ seg_rows, const int* __restrict__ seg_src,
                     const int* __restrict__ seg_src_row, const int* __restrict__ seg_dst_row, int n_seg,
                     __nv_bfloat16* __restrict__ dst, int H) {
  const int nvec = H >> 3;
  for (int g = 0; g < n_seg; ++g) {
    const int rows = seg_rows[g];
    if (rows == 0) continue;
    const uint4* s = reinterpret_cast<const uint4*>(pp.src[seg_src[g]] + (size_t)seg_src_row[g] * H);
    uint4* d = reinterpret_cast<uint4*>(dst + (size_t)seg_dst_row[g] * H);
    for (int r = blockIdx.x; r < rows; r += gridDim.x)
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) d[(size_t)r * nvec + v] = s[(size_t)r * nvec + v];
  }
}

}  // namespace trlb

using namespace trlb;

TRLB_API int trlb_moe_pull_rows(const unsigned long long* src_bases, int n_src, const int* seg_rows, const int* seg_src,
                                const int* seg_src_row, const int* seg_dst_row, int n_seg, void* dst, int H,
                                cudaStream_t st) {
  if (n_seg <= 0) return 0;
  if (H % 8 || n_src < 1 || n_src > 8) return -141;
  PullParams pp;
  for (int i = 0; i < 8; ++i) pp.src[i] = reinterpret_cast<const __nv_bfloat16*>(src_bases[i < n_src ? i : 0]);
  moe_pull_rows_kernel<<<148 * 4, 256, 0, st>>>(pp, seg_rows, seg_src, seg_src_row, seg_dst_row, n_seg,
                                                (__nv_bfloat16*)dst, H);
  return (int)cudaGetLastError();
}

TRLB_API int trlb_moe_combine(const void* y, const int* inv, const float* w, void* out, int T, int k, int H,
                              cudaStream_t st) {
  if (T == 0) return 0;
  if (H % 8) return -140;
  int threads = H / 8 < 256 ? ((H / 8 + 31) / 32) * 32 : 256;
  moe_combine_kernel<<<T, threads, 0, st>>>((const __nv_bfloat16*)y, inv, w, (__nv_bfloat16*)out, T, k, H);
  return (int)cudaGetLastError();
}
