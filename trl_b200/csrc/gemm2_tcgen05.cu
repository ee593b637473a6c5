// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): two SMs work on one 256 x 256 output tile.
//
//     C[M,N] = op(A) . op(B)^T      operands K-major or MN-major as in gemm_tcgen05.cu (forward, dgrad, wgrad)
//
// Why pairs: with one CTA per 128 x 256 tile every MMA of 16 k-columns reads 4 KB of A and 8 KB of B from shared
// memory; in a pair each CTA stages its own 128 rows of A and only HALF of the B tile (128 of the 256 columns), and the
// tensor cores of both SMs read both halves.  Shared-memory traffic and TMA traffic per SM drop by a third, and a
// stage is 32 KB instead of 48 KB, so the ring is seven stages deep instead of four.
//
// Roles per CTA (192 threads): warp 0 = TMA producer (its own A rows and its half of B; completion is counted on the
// LEADER's barrier, CTA rank 0 of the pair), warp 1 = TMEM allocation in both CTAs and, in the leader only, the MMA
// issue for the pair (tcgen05.mma.cta_group::2 writes 128 accumulator rows into each CTA's tensor memory), warps 2-5 =
// epilogue of the CTA's own 128 rows.  Barriers: full[s] (leader's; one arrival + the bytes of both CTAs), empty[s]
// and tfull[a] (one per CTA; the leader's tcgen05.commit arrives on both with a CTA mask), tempty[a] (leader's; the
// eight epilogue warps of the pair arrive on it, the follower's through the cluster address of the barrier).
// Every wait is bounded; the two cluster barriers (after set-up, before exit) are reached by both CTAs on every path.
//
// Plain-store epilogue only (bias optional): this is the kernel of the decoder linears in training.  The fused
// epilogues (lm_head statistics, all-gather) stay on the one-CTA kernel.
#include "common.cuh"

namespace trlb {

constexpr int P_BM = 128;   // rows of A per CTA (256 per pair)
constexpr int P_BN = 256;   // columns of the pair's tile; each CTA stages P_BN / 2 of them
constexpr int P_BK = 64, P_STAGES = 7;
constexpr uint32_t P_A_BYTES = P_BM * P_BK * 2, P_B_BYTES = (P_BN / 2) * P_BK * 2, P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int P_THREADS = 192;
constexpr size_t P_SMEM = P_STAGES * P_STAGE_BYTES + 1024 + 256;

struct PairGemmParams {
  int M, N, K;
  int a_mn, b_mn;
  int m_tiles, n_tiles, k_blocks;  // m_tiles counts 256-row tiles
  __nv_bfloat16* C;
  long long ldc;
  const __nv_bfloat16* bias;
  int* status;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of a CTA pair: the data lands in this CTA's shared memory, the bytes are counted on `bar_cluster`
// (a cluster address: the leader's barrier).  No multicast: each CTA fetches its own tile.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(m), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D (128 rows in each CTA's tensor memory) (+)= A (128 rows from each CTA) * B (N / 2 columns from each CTA)
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((uint16_t)3)
      : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const PairGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P_STAGES * P_STAGE_BYTES);
  uint64_t* full_bar = bars;                        // [P_STAGES]  used in the leader
  uint64_t* empty_bar = bars + P_STAGES;            // [P_STAGES]  one per CTA
  uint64_t* tfull_bar = bars + 2 * P_STAGES;        // [2]         one per CTA
  uint64_t* tempty_bar = bars + 2 * P_STAGES + 2;   // [2]         used in the leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * P_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int total_items = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
    tc_fence_before();
  }
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised and both allocations are done before either is used
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = pair; item < total_items && ok; item += n_pairs) {
        const int mt = item % p.m_tiles, nt = item / p.m_tiles;
        const int row0 = mt * 2 * P_BM + (int)rank * P_BM;        // this CTA's rows of A / C
        const int col0 = nt * P_BN + (int)rank * (P_BN / 2);      // this CTA's half of the B tile
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 900 + stage)) { ok = false; break; }
          uint8_t* sa = tiles + stage * P_STAGE_BYTES;
          uint8_t* sb = sa + P_A_BYTES;
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * P_STAGE_BYTES);
          if (p.a_mn) {
#pragma unroll
            for (int b = 0; b < P_BM / 64; ++b) tma_load_2d_pair(sa + b * 8192, &tmap_a, bar, row0 + b * 64, kb * P_BK);
          } else {
            tma_load_2d_pair(sa, &tmap_a, bar, kb * P_BK, row0);
          }
          if (p.b_mn) {
#pragma unroll
            for (int b = 0; b < P_BN / 128; ++b) tma_load_2d_pair(sb + b * 8192, &tmap_b, bar, col0 + b * 64, kb * P_BK);
          } else {
            tma_load_2d_pair(sb, &tmap_b, bar, kb * P_BK, col0);
          }
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      const uint32_t idesc = umma_idesc_bf16_major(2 * P_BM, P_BN, p.a_mn != 0, p.b_mn != 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int item = pair; item < total_items && ok; item += n_pairs) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, 910 + acc)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tacc = tmem_base + (uint32_t)acc * P_BN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 920 + stage)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * P_STAGE_BYTES);
          const uint64_t adesc = p.a_mn ? umma_desc_mnmajor_sw128(sa, 8192) : umma_desc_kmajor_sw128(sa);
          const uint64_t bdesc = p.b_mn ? umma_desc_mnmajor_sw128(sa + P_A_BYTES, 8192) : umma_desc_kmajor_sw128(sa + P_A_BYTES);
          const uint32_t astep = p.a_mn ? 128u : 2u, bstep = p.b_mn ? 128u : 2u;
#pragma unroll
          for (int kk = 0; kk < P_BK / 16; ++kk)
            umma_bf16_ss_pair(tacc, adesc + astep * kk, bdesc + bstep * kk, idesc, (kb | kk) != 0);
          umma_commit_pair(&empty_bar[stage]);  // both producers may refill this stage once the MMAs have read it
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(&tfull_bar[acc]);  // accumulator complete in both CTAs
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue warps 2..5 (both CTAs): this CTA's 128 rows ----------------
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int item = pair; item < total_items && ok; item += n_pairs) {
      const int mt = item % p.m_tiles, nt = item / p.m_tiles;
      const int row = mt * 2 * P_BM + (int)rank * P_BM + r;
      const bool row_ok = row < p.M;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, 930 + acc)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tacc = tmem_base + (uint32_t)acc * P_BN + ((uint32_t)(quarter * 32) << 16);
      const int col0 = nt * P_BN;
#pragma unroll 1
      for (int c = 0; c < P_BN; c += 32) {
        float v[32];
        tmem_ld_32x32(tacc + c, v);
        tmem_ld_wait();
        const int cbase = col0 + c;
        if (row_ok && cbase < p.N) {
          __nv_bfloat16* dst = p.C + (long long)row * p.ldc + cbase;
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (cbase + i < p.N) v[i] += __bfloat162float(p.bias[cbase + i]);
          }
          if (cbase + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 o;
              o.x = pack_bf16(v[i], v[i + 1]);
              o.y = pack_bf16(v[i + 2], v[i + 3]);
              o.z = pack_bf16(v[i + 4], v[i + 5]);
              o.w = pack_bf16(v[i + 6], v[i + 7]);
              *reinterpret_cast<uint4*>(dst + i) = o;
            }
          } else {
            for (int i = 0; i < 32; ++i)
              if (cbase + i < p.N) dst[i] = __float2bfloat16(v[i]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));  // the leader's barrier
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  __syncthreads();
  if (*abort_flag) {  // a role gave up: let copies in flight land before the shared memory goes away
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();  // the peer no longer reads this CTA's tiles or signals its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

}  // namespace trlb

using namespace trlb;

// C[M,N] (bf16, row stride ldc) = op(A) . op(B)^T (+ bias[N]); a_mn / b_mn as in trlb_gemm_bf16.
TRLB_API int trlb_gemm_pair_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                                 long long lda, long long ldb, long long ldc, int a_mn, int b_mn, int* status,
                                 cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) != 0 || (ldb % 8) != 0) return -150;
  if ((!a_mn || !b_mn) && (K % 8) != 0) return -150;
  if ((a_mn && (M % 8)) || (b_mn && (N % 8))) return -150;
  CUtensorMap ta, tb;
  int r = a_mn ? trlb_host::make_tmap_2d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, P_BK, 64)
               : trlb_host::make_tmap_2d_bf16(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, P_BM, P_BK);
  if (r) return -151;
  r = b_mn ? trlb_host::make_tmap_2d_bf16(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, P_BK, 64)
           : trlb_host::make_tmap_2d_bf16(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, P_BN / 2, P_BK);
  if (r) return -152;
  PairGemmParams p = {};
  p.M = M; p.N = N; p.K = K; p.a_mn = a_mn ? 1 : 0; p.b_mn = b_mn ? 1 : 0;
  p.m_tiles = (M + 2 * P_BM - 1) / (2 * P_BM);
  p.n_tiles = (N + P_BN - 1) / P_BN;
  p.k_blocks = (K + P_BK - 1) / P_BK;
  p.C = (__nv_bfloat16*)C; p.ldc = ldc; p.bias = (const __nv_bfloat16*)bias; p.status = status;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P_SMEM);
    attr_set = true;
  }
  const int items = p.m_tiles * p.n_tiles;
  // persistent pairs: as many as the GPU can hold at once (a GPC with an odd number of free SMs leaves one out)
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(trlb_host::sm_count() / 2 * 2);
    cfg.blockDim = dim3(P_THREADS);
    cfg.dynamicSmemBytes = P_SMEM;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel, &cfg) != cudaSuccess || n < 1) {
      (void)cudaGetLastError();
      n = trlb_host::sm_count() / 2;
    }
    max_pairs = n;
  }
  int pairs = max_pairs;
  if (items < pairs) pairs = items;
  gemm_pair_kernel<<<2 * pairs, P_THREADS, P_SMEM, stream>>>(ta, tb, p);
  return (int)cudaGetLastError();
}
