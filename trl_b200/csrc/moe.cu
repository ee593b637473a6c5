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

// Backward of the weighted combine, one permuted row per CTA iteration: with (t, j) = the (token, choice) that row r
// holds (order[r] = t * k + j),
//     d_y[r, :] = w[t, j] * d_out[t, :]          (gradient of the expert output row)
//     d_w[t, j] = <d_out[t, :], y[r, :]>         (gradient of the routing weight)
// d_out is read once per choice (k rows share a token; the repeats hit L2), y once, d_y written once.
__global__ void __launch_bounds__(256)
moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ d_out, const __nv_bfloat16* __restrict__ y,
                       const long long* __restrict__ order, const float* __restrict__ w,
                       __nv_bfloat16* __restrict__ d_y, float* __restrict__ d_w, long long rows, int k, int H) {
  const int nvec = H >> 3;
  __shared__ float part[8];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const long long flat = order[r];
    const long long t = flat / k;
    const float wj = w[flat];
    float dot = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 g = reinterpret_cast<const uint4*>(d_out + (size_t)t * H)[v];
      const uint4 yy = reinterpret_cast<const uint4*>(y + (size_t)r * H)[v];
      const uint32_t gq[4] = {g.x, g.y, g.z, g.w}, yq[4] = {yy.x, yy.y, yy.z, yy.w};
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = unpack_bf16(gq[i]), b = unpack_bf16(yq[i]);
        dot = fmaf(a.x, b.x, fmaf(a.y, b.y, dot));
        o[i] = pack_bf16(wj * a.x, wj * a.y);
      }
      reinterpret_cast<uint4*>(d_y + (size_t)r * H)[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    dot = warp_sum(dot);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = dot;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
      for (int i = 0; i < (int)(blockDim.x >> 5); ++i) s += part[i];
      d_w[flat] = s;
    }
    __syncthreads();
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

// ------------------------------------------------------------------------------------------------
// Router load-balancing loss  E * sum_e f_e * P_e  in one pass (the reference computes it from one-hot tensors of
// shape [tokens, k, experts], transformers' load_balancing_loss_func reached through trl/trainer/sft_trainer.py:357-378):
// f_e = routed choices to expert e / valid tokens, P_e = mean router probability of expert e over valid tokens.
// Every block reduces its slice of tokens into shared memory (probability columns in registers, counts with
// shared-memory atomics), adds the slice to a small global accumulator, and the last block to arrive forms the loss,
// writes f (needed by the backward: dL/dP[n, e] = E * f_e * mask_n / valid) and leaves the accumulator zeroed.
// ------------------------------------------------------------------------------------------------
namespace trlb {

constexpr int AUX_THREADS = 256;
constexpr int AUX_MAX_E = 1024;

template <typename PT>
__global__ void __launch_bounds__(AUX_THREADS)
moe_aux_loss_kernel(const PT* __restrict__ probs, const long long* __restrict__ idx, const float* __restrict__ mask,
                    int N, int E, int K, int rows_per_block, float* __restrict__ acc /* [2E + 2] */,
                    float* __restrict__ loss, float* __restrict__ f_out /* [E] */, float* __restrict__ valid_out) {
  __shared__ float ps[AUX_MAX_E], cnt[AUX_MAX_E];
  __shared__ float msum_s;
  __shared__ unsigned ticket_s;
  const int t = threadIdx.x;
  for (int e = t; e < E; e += AUX_THREADS) { ps[e] = 0.f; cnt[e] = 0.f; }
  if (t == 0) msum_s = 0.f;
  __syncthreads();
  const int r0 = blockIdx.x * rows_per_block, r1 = min(N, r0 + rows_per_block);
  // probability columns: thread (row group, column) walks its rows; up to 4 columns per thread
  const int cols = E < AUX_THREADS ? E : AUX_THREADS, rgroups = AUX_THREADS / cols;
  const int my_col = t % cols, my_rg = t / cols;
  float part[4] = {0.f, 0.f, 0.f, 0.f};
  if (my_rg < rgroups) {
    for (int r = r0 + my_rg; r < r1; r += rgroups) {
      const float m = mask ? mask[r] : 1.f;
      if (m == 0.f) continue;
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const int e = my_col + s * cols;
        if (e < E) part[s] += m * (float)probs[(size_t)r * E + e];
      }
    }
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int e = my_col + s * cols;
      if (e < E && part[s] != 0.f) atomicAdd(&ps[e], part[s]);
    }
  }
  // routed choices
  float ml = 0.f;
  for (int i = r0 * K + t; i < r1 * K; i += AUX_THREADS) {
    const int r = i / K;
    const float m = mask ? mask[r] : 1.f;
    const long long e = idx[i];
    if (m != 0.f && e >= 0 && e < E) atomicAdd(&cnt[(int)e], m);
  }
  for (int r = r0 + t; r < r1; r += AUX_THREADS) ml += mask ? mask[r] : 1.f;
  ml = warp_sum(ml);
  if ((t & 31) == 0 && ml != 0.f) atomicAdd(&msum_s, ml);
  __syncthreads();
  for (int e = t; e < E; e += AUX_THREADS) {
    if (ps[e] != 0.f) atomicAdd(&acc[e], ps[e]);
    if (cnt[e] != 0.f) atomicAdd(&acc[E + e], cnt[e]);
  }
  if (t == 0 && msum_s != 0.f) atomicAdd(&acc[2 * E], msum_s);
  __threadfence();
  __syncthreads();
  if (t == 0) ticket_s = atomicAdd(reinterpret_cast<unsigned*>(&acc[2 * E + 1]), 1u);
  __syncthreads();
  if (ticket_s != gridDim.x - 1) return;
  // last block: everything has been added
  __threadfence();
  const float valid = fmaxf(__ldcg(&acc[2 * E]), 1.f);
  float l = 0.f;
  for (int e = t; e < E; e += AUX_THREADS) {
    const float p = __ldcg(&acc[e]) / valid, f = __ldcg(&acc[E + e]) / valid;
    f_out[e] = f;
    l += f * p;
    acc[e] = 0.f;
    acc[E + e] = 0.f;
  }
  l = warp_sum(l);
  __syncthreads();
  if (t == 0) msum_s = 0.f;
  __syncthreads();
  if ((t & 31) == 0) atomicAdd(&msum_s, l);
  __syncthreads();
  if (t == 0) {
    *loss = msum_s * (float)E;
    *valid_out = valid;
    acc[2 * E] = 0.f;
    *reinterpret_cast<unsigned*>(&acc[2 * E + 1]) = 0u;
  }
}

}  // namespace trlb

// probs [N, E] (fp32 or bf16), idx [N, K] int64, mask [N] fp32 or null.  acc: 2E + 2 zero-initialised floats of scratch
// (left zeroed).  Outputs: loss (scalar), f_out [E] (routed fraction per expert), valid_out (number of valid tokens).
TRLB_API int trlb_moe_aux_loss(const void* probs, int probs_bf16, const long long* idx, const float* mask, int N, int E,
                               int K, float* acc, float* loss, float* f_out, float* valid_out, cudaStream_t st) {
  if (E <= 0 || E > trlb::AUX_MAX_E || K <= 0) return -1;
  if (N <= 0) {
    cudaMemsetAsync(loss, 0, sizeof(float), st);
    return (int)cudaGetLastError();
  }
  int blocks = (N + 63) / 64;
  const int cap = 2 * trlb_host::sm_count();
  if (blocks > cap) blocks = cap;
  const int rows_per_block = (N + blocks - 1) / blocks;
  blocks = (N + rows_per_block - 1) / rows_per_block;
  if (probs_bf16)
    trlb::moe_aux_loss_kernel<__nv_bfloat16><<<blocks, trlb::AUX_THREADS, 0, st>>>(
        (const __nv_bfloat16*)probs, idx, mask, N, E, K, rows_per_block, acc, loss, f_out, valid_out);
  else
    trlb::moe_aux_loss_kernel<float><<<blocks, trlb::AUX_THREADS, 0, st>>>((const float*)probs, idx, mask, N, E, K,
                                                                           rows_per_block, acc, loss, f_out, valid_out);
  return (int)cudaGetLastError();
}

// d_out [T, H] bf16, y [rows, H] bf16 (expert-sorted), order [rows] int64 (flat (token, choice) index of every row),
// w [T * k] fp32 -> d_y [rows, H] bf16, d_w [T * k] fp32 (every entry written: order is a permutation).
TRLB_API int trlb_moe_combine_bwd(const void* d_out, const void* y, const long long* order, const float* w, void* d_y,
                                  float* d_w, long long rows, int k, int H, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (H % 8) return -142;
  const long long grid = rows < 148LL * 16 ? rows : 148LL * 16;
  moe_combine_bwd_kernel<<<(int)grid, 256, 0, st>>>((const __nv_bfloat16*)d_out, (const __nv_bfloat16*)y, order, w,
                                                    (__nv_bfloat16*)d_y, d_w, rows, k, H);
  return (int)cudaGetLastError();
}
