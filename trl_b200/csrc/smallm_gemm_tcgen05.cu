// Weight-streaming GEMM for decode batches (at most 64 rows) on the 5th-generation tensor cores.
//
//     Y[b, n] += sum_k X[b, k] * W[n, k]         B <= 64 rows of X, W [N, K] row-major, Y fp32 [B, N]
//
// With so few rows the cost is reading W once, so the kernel is laid out for bandwidth: the operands are swapped
// (the 128-row weight slab is the M operand of the MMA, the batch is the N = 64 operand), the reduction dimension is
// split over CTAs until every SM streams a piece of W (grid = N/128 slabs x K splits), an 8-stage TMA ring keeps
// ~190 KB in flight per SM, and partial sums are added to the fp32 output with red.global (lanes = consecutive n,
// so each warp-level reduction is a 128-byte line).  The consumer of Y (residual add + RMSNorm) reads the fp32 sums
// and clears them, so no separate zeroing or conversion kernel runs.
//
// The reference has no counterpart (decode GEMMs belong to vLLM there).
#include "common.cuh"

namespace trlb {

constexpr int SM_BM = 128, SM_BN = 64, SM_BK = 64, SM_STAGES = 8;
constexpr uint32_t SM_A_BYTES = SM_BM * SM_BK * 2, SM_B_BYTES = SM_BN * SM_BK * 2, SM_STAGE = SM_A_BYTES + SM_B_BYTES;
constexpr int SM_THREADS = 192;
constexpr size_t SM_SMEM = SM_STAGES * SM_STAGE + 1024 + 256;

struct SmallMParams {
  int B, N, K, k_blocks, splits;
  float* Y;          // [B, ldy] fp32, accumulated into
  long long ldy;
  const __nv_bfloat16* bias;  // added once (by split 0) or null
  int* status;
};

__global__ void __launch_bounds__(SM_THREADS, 1)
smallm_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   const SmallMParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM_STAGES * SM_STAGE);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + SM_STAGES;
  uint64_t* done_bar = bars + 2 * SM_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * SM_STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slab = blockIdx.x, split = blockIdx.y;
  const int per = (p.k_blocks + p.splits - 1) / p.splits;
  const int kb0 = split * per, kb1 = min(p.k_blocks, kb0 + per);

  if (threadIdx.x == 0) {
    for (int s = 0; s < SM_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(done_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (kb1 > kb0) {
    if (warp == 0) {
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 900 + stage)) break;
          uint8_t* sa = smem + stage * SM_STAGE;
          mbar_expect_tx(&full_bar[stage], SM_STAGE);
          tma_load_2d(sa, &tmap_w, &full_bar[stage], kb * SM_BK, slab * SM_BM);
          tma_load_2d(sa + SM_A_BYTES, &tmap_x, &full_bar[stage], kb * SM_BK, 0);
          if (++stage == SM_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      if (lane == 0) {
        constexpr uint32_t idesc = umma_idesc_bf16(SM_BM, SM_BN);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 910 + stage)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * SM_STAGE);
          const uint64_t adesc = umma_desc_kmajor_sw128(sa);
          const uint64_t bdesc = umma_desc_kmajor_sw128(sa + SM_A_BYTES);
#pragma unroll
          for (int kk = 0; kk < SM_BK / 16; ++kk)
            umma_bf16_ss(tmem_base, adesc + 2 * kk, bdesc + 2 * kk, idesc, (kb != kb0) || kk != 0);
          umma_commit(&empty_bar[stage]);
          if (++stage == SM_STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(done_bar);
      }
      __syncwarp();
    } else {
      const int quarter = warp & 3;
      const int n = slab * SM_BM + quarter * 32 + lane;  // this thread's output column (a row of W)
      if (mbar_wait(done_bar, 0, abort_flag, p.status, 920)) {
        tc_fence_after();
        const uint32_t tacc = tmem_base + ((uint32_t)(quarter * 32) << 16);
        float bias = 0.f;
        if (p.bias != nullptr && split == 0 && n < p.N) bias = __bfloat162float(p.bias[n]);
#pragma unroll 1
        for (int c = 0; c < SM_BN; c += 32) {
          float v[32];
          tmem_ld_32x32(tacc + c, v);
          tmem_ld_wait();
          if (n < p.N) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c + i < p.B) atomicAdd(p.Y + (long long)(c + i) * p.ldy + n, v[i] + bias);
          }
        }
        tc_fence_before();
      }
    }
  }
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 64);
  }
}

}  // namespace trlb

using namespace trlb;

// X [B, K] bf16 (row stride ldx), W [N, K] bf16 (row stride ldw), Y [B, N] fp32 (row stride ldy) is accumulated into:
// the caller provides zeros (or a value to add to).  B <= 64.
TRLB_API int trlb_smallm_gemm_bf16(const void* X, const void* W, const void* bias, float* Y, int B, int N, int K,
                                   long long ldx, long long ldw, long long ldy, int* status, cudaStream_t st) {
  if (B <= 0 || N <= 0 || K <= 0) return 0;
  if (B > SM_BN || (K % 8) != 0 || (ldx % 8) != 0 || (ldw % 8) != 0) return -150;
  CUtensorMap tw, tx;
  if (trlb_host::make_tmap_2d_bf16(&tw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, SM_BM, SM_BK)) return -151;
  if (trlb_host::make_tmap_2d_bf16(&tx, X, (uint64_t)B, (uint64_t)K, (uint64_t)ldx, SM_BN, SM_BK)) return -152;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(smallm_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SM_SMEM);
    attr_set = true;
  }
  SmallMParams p;
  p.B = B; p.N = N; p.K = K; p.k_blocks = (K + SM_BK - 1) / SM_BK;
  const int slabs = (N + SM_BM - 1) / SM_BM;
  int splits = (trlb_host::sm_count() + slabs - 1) / slabs;  // about one CTA per SM
  if (splits > p.k_blocks / 4) splits = p.k_blocks / 4 > 0 ? p.k_blocks / 4 : 1;  // at least 4 K blocks per CTA
  p.splits = splits;
  p.Y = Y; p.ldy = ldy; p.bias = (const __nv_bfloat16*)bias; p.status = status;
  smallm_gemm_kernel<<<dim3(slabs, splits), SM_THREADS, SM_SMEM, st>>>(tw, tx, p);
  return (int)cudaGetLastError();
}
