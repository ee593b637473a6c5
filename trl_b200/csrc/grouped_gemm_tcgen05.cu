// Grouped (per-expert) bf16 GEMM on the 5th-generation tensor cores for mixture-of-experts layers.
//
//     C[r, :] = A[r, :] . W[e(r)]^T      rows of A are sorted by expert; offsets[e] .. offsets[e+1] belong to expert e
//
// Same persistent warp-specialised pipeline as the dense GEMM (warp 0 TMA producer, warp 1 tcgen05.mma issuer,
// warps 2-5 epilogue, 128x256x64 tiles, 4-stage ring, two TMEM accumulators).  What differs:
//   * the tile list is derived on the device from `offsets` (token counts per expert are only known on the GPU, and
//     the launch must be capturable in a CUDA graph): every CTA builds the prefix of 128-row tiles per expert in shared
//     memory and maps its work items through it;
//   * the weight tile comes from a 3D tensor map (K, N, experts); the activation tile starts at the expert's first
//     row, wherever that is; rows of the tile that belong to the next expert are computed and thrown away;
//   * segment mode (expert parallelism): a segment is (local expert, source rank); its activation rows are read with TMA
//     straight from the source rank's buffer over NVLink (no cluster sharing of those tiles), and the output rows are
//     stored straight into a destination rank's buffer, so the dispatch all-to-all rides on the loads of the first GEMM
//     and the combine all-to-all on the stores of the second;
//   * optional SwiGLU epilogue for the gate/up projection: the B tile is 128 gate rows + the matching 128 up rows, the
//     epilogue writes silu(gate) * up, so the [tokens, 2I] intermediate never reaches memory.
//
// Replaces the per-expert loop of transformers' MoE blocks that the reference trains through
// (trl/trainer/grpo_trainer.py forward of Qwen3-MoE style models).
#include "common.cuh"

namespace trlb {

constexpr int GBM = 128, GBN = 256, GBK = 64, GSTAGES = 4;
constexpr uint32_t GA_BYTES = GBM * GBK * 2, GB_BYTES = GBN * GBK * 2, GSTAGE_BYTES = GA_BYTES + GB_BYTES;
constexpr int G_THREADS = 192;
constexpr int G_MAX_EXPERTS = 1024;
constexpr size_t G_SMEM = GSTAGES * GSTAGE_BYTES + 1024 + 256 + (G_MAX_EXPERTS + 1) * 4;

struct TmapArray {
  CUtensorMap m[8];
};

struct GroupedParams {
  int E, N, K, n_tiles, k_blocks;
  int swiglu;          // 1: W is [E, 2*N, K] (gate rows then up rows), C gets N columns
  int b_mn;            // 1: W is [E, K, N] (the weight of the forward pass read transposed: input gradient)
  const int* offsets;  // [E + 1] row offsets into A / C (plain mode)
  __nv_bfloat16* C;
  long long ldc;
  int* status;
  // segment mode (n_seg > 0): E counts segments; per segment: rows, A source (tensor-map index) and first row,
  // C destination (index into c_dst) and first row, weight index
  int n_seg;
  const int* seg_rows;
  const int* seg_a_src;
  const int* seg_a_row;
  const int* seg_c_dst;
  const int* seg_c_row;
  const int* seg_w;
  __nv_bfloat16* c_dst[8];
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

__global__ void __launch_bounds__(G_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ TmapArray tmaps_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GroupedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GSTAGES * GSTAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + GSTAGES;
  uint64_t* tfull_bar = bars + 2 * GSTAGES;
  uint64_t* tempty_bar = bars + 2 * GSTAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * GSTAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* mt_prefix = reinterpret_cast<int*>(tmem_slot + 4);  // [E + 1] prefix of 128-row tiles per expert

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < GSTAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmaps_a.m[0]);
    tma_prefetch_desc(&tmap_b);
  }
  // 128-row tiles per group (expert or segment), then their prefix
  for (int e = threadIdx.x; e < p.E; e += G_THREADS) {
    const int cnt = p.n_seg ? p.seg_rows[e] : p.offsets[e + 1] - p.offsets[e];
    mt_prefix[e + 1] = (cnt + GBM - 1) / GBM;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    mt_prefix[0] = 0;
    for (int e = 0; e < p.E; ++e) mt_prefix[e + 1] += mt_prefix[e];
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_items = mt_prefix[p.E] * p.n_tiles;

  // item -> (group, first A row, valid rows, n tile, first C row)
  auto decode = [&](int item, int& e, int& row0, int& rows, int& nt, int& crow0) {
    const int mt = item / p.n_tiles;
    nt = item % p.n_tiles;
    int lo = 0, hi = p.E;  // largest e with mt_prefix[e] <= mt
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (mt_prefix[mid] <= mt) lo = mid; else hi = mid;
    }
    e = lo;
    const int m_off = (mt - mt_prefix[e]) * GBM;
    if (p.n_seg) {
      row0 = p.seg_a_row[e] + m_off;
      crow0 = p.seg_c_row[e] + m_off;
      rows = min(GBM, p.seg_rows[e] - m_off);
    } else {
      row0 = p.offsets[e] + m_off;
      crow0 = row0;
      rows = min(GBM, p.offsets[e + 1] - row0);
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        int e, row0, rows, nt, crow0;
        decode(item, e, row0, rows, nt, crow0);
        const CUtensorMap* ta = &tmaps_a.m[p.n_seg ? p.seg_a_src[e] : 0];  // segment mode: possibly a peer's buffer
        const int we = p.n_seg ? p.seg_w[e] : e;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 800 + stage)) { ok = false; break; }
          uint8_t* sa = tiles + stage * GSTAGE_BYTES;
          uint8_t* sb = sa + GA_BYTES;
          mbar_expect_tx(&full_bar[stage], GSTAGE_BYTES);
          tma_load_2d(sa, ta, &full_bar[stage], kb * GBK, row0);
          if (p.b_mn) {  // [64 k-rows x 64 columns] boxes, one per 64 output columns
#pragma unroll
            for (int b = 0; b < GBN / 64; ++b)
              tma_load_3d(sb + b * 8192, &tmap_b, &full_bar[stage], nt * GBN + b * 64, kb * GBK, we);
          } else if (p.swiglu) {  // 128 gate rows, then the 128 up rows of the same output columns
            tma_load_3d(sb, &tmap_b, &full_bar[stage], kb * GBK, nt * 128, we);
            tma_load_3d(sb + GB_BYTES / 2, &tmap_b, &full_bar[stage], kb * GBK, p.N + nt * 128, we);
          } else {
            tma_load_3d(sb, &tmap_b, &full_bar[stage], kb * GBK, nt * GBN, we);
            tma_load_3d(sb + GB_BYTES / 2, &tmap_b, &full_bar[stage], kb * GBK, nt * GBN + 128, we);
          }
          if (++stage == GSTAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16_major(GBM, GBN, false, p.b_mn != 0);
      const uint32_t bstep = p.b_mn ? 128u : 2u;  // K step of 16: 32 bytes in a K-major atom, 16 rows of 128 bytes MN-major
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, 810 + acc)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tacc = tmem_base + (uint32_t)acc * GBN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 820 + stage)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * GSTAGE_BYTES);
          const uint64_t adesc = umma_desc_kmajor_sw128(sa);
          const uint64_t bdesc = p.b_mn ? umma_desc_mnmajor_sw128(sa + GA_BYTES, 8192) : umma_desc_kmajor_sw128(sa + GA_BYTES);
#pragma unroll
          for (int kk = 0; kk < GBK / 16; ++kk)
            umma_bf16_ss(tacc, adesc + 2 * kk, bdesc + bstep * kk, idesc, (kb | kk) != 0);
          umma_commit(&empty_bar[stage]);
          if (++stage == GSTAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      int e, row0, rows, nt, crow0;
      decode(item, e, row0, rows, nt, crow0);
      __nv_bfloat16* cbase = p.n_seg ? p.c_dst[p.seg_c_dst[e]] : p.C;  // segment mode: possibly a peer's buffer
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, 830 + acc)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tacc = tmem_base + (uint32_t)acc * GBN + ((uint32_t)(quarter * 32) << 16);
      const bool row_ok = r < rows;
      if (p.swiglu) {
        const int col0 = nt * 128;
#pragma unroll 1
        for (int c = 0; c < 128; c += 32) {
          float g[32], u[32];
          tmem_ld_32x32(tacc + c, g);
          tmem_ld_32x32(tacc + 128 + c, u);
          tmem_ld_wait();
          if (row_ok && col0 + c < p.N) {
            __nv_bfloat16* dst = cbase + (long long)(crow0 + r) * p.ldc + col0 + c;
            if (col0 + c + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 o;
                o.x = pack_bf16(silu_f(g[i]) * u[i], silu_f(g[i + 1]) * u[i + 1]);
                o.y = pack_bf16(silu_f(g[i + 2]) * u[i + 2], silu_f(g[i + 3]) * u[i + 3]);
                o.z = pack_bf16(silu_f(g[i + 4]) * u[i + 4], silu_f(g[i + 5]) * u[i + 5]);
                o.w = pack_bf16(silu_f(g[i + 6]) * u[i + 6], silu_f(g[i + 7]) * u[i + 7]);
                *reinterpret_cast<uint4*>(dst + i) = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + c + i < p.N) dst[i] = __float2bfloat16(silu_f(g[i]) * u[i]);
            }
          }
        }
      } else {
        const int col0 = nt * GBN;
#pragma unroll 1
        for (int c = 0; c < GBN; c += 32) {
          float v[32];
          tmem_ld_32x32(tacc + c, v);
          tmem_ld_wait();
          if (row_ok && col0 + c < p.N) {
            __nv_bfloat16* dst = cbase + (long long)(crow0 + r) * p.ldc + col0 + c;
            if (col0 + c + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
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
                if (col0 + c + i < p.N) dst[i] = __float2bfloat16(v[i]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
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
    tmem_dealloc(tmem_base, 512);
  }
}


// ---------------------------------------------------------------------------------------------------------------------
// Grouped weight gradient:  dW[e] = G[rows of e]^T . X[rows of e]     (dW[e] is [Nw, Kw], G [rows, Nw], X [rows, Kw])
//
// The contraction runs over the rows of expert e, so both operands are MN-major (a TMA box is [64 rows x 64 columns],
// rows = reduction dimension) and nothing is transposed in memory.  One item = (expert, 128 x 256 tile of dW[e]); its
// K loop walks the expert's rows in blocks of 64, starting at the expert's first row wherever that is.  The last block
// of an expert runs into the rows of the next one: the MMA warp clears those rows of the G tile in shared memory
// before it issues (a zero row of either operand removes the term), which costs a few hundred 16-byte stores per item.
// An expert without rows gets zeros.
// ---------------------------------------------------------------------------------------------------------------------
struct GroupedWgradParams {
  int E, Nw, Kw, m_tiles, n_tiles;
  const int* offsets;
  __nv_bfloat16* dW;
  int* status;
};

__global__ void __launch_bounds__(G_THREADS, 1)
grouped_wgrad_kernel(const __grid_constant__ CUtensorMap tmap_g, const __grid_constant__ CUtensorMap tmap_x,
                     const GroupedWgradParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GSTAGES * GSTAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + GSTAGES;
  uint64_t* tfull_bar = bars + 2 * GSTAGES;
  uint64_t* tempty_bar = bars + 2 * GSTAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * GSTAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < GSTAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_g);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int per_e = p.m_tiles * p.n_tiles;
  const int total_items = p.E * per_e;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const int e = item / per_e, mt = (item % per_e) / p.n_tiles, nt = item % p.n_tiles;
        const int r0 = p.offsets[e], cnt = p.offsets[e + 1] - r0;
        const int k_blocks = (cnt + GBK - 1) / GBK;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 840 + stage)) { ok = false; break; }
          uint8_t* sa = tiles + stage * GSTAGE_BYTES;
          uint8_t* sb = sa + GA_BYTES;
          mbar_expect_tx(&full_bar[stage], GSTAGE_BYTES);
#pragma unroll
          for (int b = 0; b < GBM / 64; ++b)
            tma_load_2d(sa + b * 8192, &tmap_g, &full_bar[stage], mt * GBM + b * 64, r0 + kb * GBK);
#pragma unroll
          for (int b = 0; b < GBN / 64; ++b)
            tma_load_2d(sb + b * 8192, &tmap_x, &full_bar[stage], nt * GBN + b * 64, r0 + kb * GBK);
          if (++stage == GSTAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // every lane follows the loop: lane 0 waits on the barriers and issues the MMAs, the whole warp clears the rows
    // past the expert's end (lane 0's wait, then the warp shuffle, orders the TMA writes before those stores)
    constexpr uint32_t idesc = umma_idesc_bf16_major(GBM, GBN, true, true);
    int stage = 0, acc = 0;
    uint32_t phase = 0, acc_phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      const int e = item / per_e;
      const int cnt = p.offsets[e + 1] - p.offsets[e];
      const int k_blocks = (cnt + GBK - 1) / GBK;
      if (lane == 0) ok = mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, 850 + acc);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();
      const uint32_t tacc = tmem_base + (uint32_t)acc * GBN;
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (lane == 0) ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 860 + stage);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        uint8_t* sa_p = tiles + stage * GSTAGE_BYTES;
        const int valid = cnt - kb * GBK;  // rows of this block that belong to the expert
        if (valid < GBK) {
          // a k-row is 128 contiguous bytes of each 64-column box (the swizzle permutes 16-byte chunks inside it)
          const int chunks = (GBK - valid) * 8;
          for (int b = 0; b < GBM / 64; ++b) {
            uint4* base = reinterpret_cast<uint4*>(sa_p + b * 8192 + valid * 128);
            for (int i = lane; i < chunks; i += 32) base[i] = make_uint4(0u, 0u, 0u, 0u);
          }
          fence_proxy_async_smem();  // generic-proxy stores -> tensor-core reads
        }
        __syncwarp();
        if (lane == 0) {
          tc_fence_after();
          const uint32_t sa = smem_u32(sa_p);
          const uint64_t adesc = umma_desc_mnmajor_sw128(sa, 8192);
          const uint64_t bdesc = umma_desc_mnmajor_sw128(sa + GA_BYTES, 8192);
#pragma unroll
          for (int kk = 0; kk < GBK / 16; ++kk)
            umma_bf16_ss(tacc, adesc + 128u * kk, bdesc + 128u * kk, idesc, (kb | kk) != 0);
          umma_commit(&empty_bar[stage]);
        }
        __syncwarp();
        if (++stage == GSTAGES) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      if (lane == 0) umma_commit(&tfull_bar[acc]);  // with no block issued this arrives at once; the epilogue writes zeros
      __syncwarp();
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      const int e = item / per_e, mt = (item % per_e) / p.n_tiles, nt = item % p.n_tiles;
      const bool empty = p.offsets[e + 1] - p.offsets[e] <= 0;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, 870 + acc)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tacc = tmem_base + (uint32_t)acc * GBN + ((uint32_t)(quarter * 32) << 16);
      const int row = mt * GBM + r, col0 = nt * GBN;
      __nv_bfloat16* out_row = p.dW + ((long long)e * p.Nw + row) * p.Kw;
#pragma unroll 1
      for (int c = 0; c < GBN; c += 32) {
        float v[32];
        tmem_ld_32x32(tacc + c, v);
        tmem_ld_wait();
        if (empty) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.f;
        }
        if (row < p.Nw && col0 + c < p.Kw) {
          __nv_bfloat16* dst = out_row + col0 + c;
          if (col0 + c + 32 <= p.Kw && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
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
              if (col0 + c + i < p.Kw) dst[i] = __float2bfloat16(v[i]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
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
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace trlb

using namespace trlb;

// A [rows, K] bf16 (row stride lda), rows sorted by expert; W [E, Nw, K] bf16 contiguous with Nw = N (plain) or
// 2 * N (swiglu: gate rows then up rows); offsets [E + 1] int32 on the device; C [rows, N] bf16 (row stride ldc).
// `rows` is the allocated row count of A and C (an upper bound of offsets[E]).
// `w_transposed` = 1: W is [E, K, N] and C[r, :] = A[r, :] . W[e] (the forward weight read transposed, for the
// input gradient); N must then be a multiple of 8 and swiglu 0.
TRLB_API int trlb_grouped_gemm_bf16(const void* A, const void* W, const int* offsets, void* C, long long rows, int E, int N,
                                    int K, long long lda, long long ldc, int swiglu, int w_transposed, int* status,
                                    cudaStream_t st) {
  if (rows <= 0 || E <= 0) return 0;
  if (E > G_MAX_EXPERTS || (K % 8) != 0 || (lda % 8) != 0) return -130;
  if (w_transposed && (swiglu || (N % 8) != 0)) return -130;
  const long long Nw = swiglu ? 2LL * N : N;
  TmapArray ta;
  CUtensorMap tb;
  int r = trlb_host::make_tmap_2d_bf16(&ta.m[0], A, (uint64_t)rows, (uint64_t)K, (uint64_t)lda, GBM, GBK);
  if (r) return -131;
  for (int i = 1; i < 8; ++i) ta.m[i] = ta.m[0];
  r = w_transposed
          ? trlb_host::make_tmap_3d_bf16(&tb, W, (uint64_t)N, (uint64_t)K, (uint64_t)E, (uint64_t)N, (uint64_t)N * K, 64, GBK, 1)
          : trlb_host::make_tmap_3d_bf16(&tb, W, (uint64_t)K, (uint64_t)Nw, (uint64_t)E, (uint64_t)K, (uint64_t)Nw * K, GBK,
                                         128, 1);
  if (r) return -132;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G_SMEM);
    attr_set = true;
  }
  GroupedParams p = {};
  p.E = E; p.N = N; p.K = K; p.swiglu = swiglu; p.b_mn = w_transposed ? 1 : 0;
  p.n_tiles = swiglu ? (N + 127) / 128 : (N + GBN - 1) / GBN;
  p.k_blocks = (K + GBK - 1) / GBK;
  p.offsets = offsets; p.C = (__nv_bfloat16*)C; p.ldc = ldc; p.status = status;
  // the number of items depends on device data: launch one CTA per SM (an idle CTA costs a few microseconds)
  long long max_items = ((rows + GBM - 1) / GBM + E) * p.n_tiles;
  int grid = trlb_host::sm_count();
  if (max_items < grid) grid = (int)max_items;
  grouped_gemm_kernel<<<grid, G_THREADS, G_SMEM, st>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

// Segment mode for expert parallelism.  a_bases[i] / c_bases[i] (i < n_bufs <= 8): buffers that the segment tables index
// (this rank's own and its peers' mappings of the same symmetric buffers); every A buffer is [a_rows, K] with row stride
// lda, every C buffer has row stride ldc.  seg_* are int32 device arrays of length n_seg; W [E_local, Nw, K].
// max_rows bounds the total number of rows over all segments (sizes the grid only).  `w_transposed`: W is
// [E_local, K, N], read as it lies (input gradient of a layer whose forward weight is W).
TRLB_API int trlb_grouped_gemm_seg_bf16(const unsigned long long* a_bases, const unsigned long long* c_bases, int n_bufs,
                                        long long a_rows, const void* W, int E_local, int n_seg, const int* seg_rows,
                                        const int* seg_a_src, const int* seg_a_row, const int* seg_c_dst,
                                        const int* seg_c_row, const int* seg_w, long long max_rows, int N, int K,
                                        long long lda, long long ldc, int swiglu, int w_transposed, int* status,
                                        cudaStream_t st) {
  if (n_seg <= 0 || max_rows <= 0) return 0;
  if (n_seg > G_MAX_EXPERTS || n_bufs < 1 || n_bufs > 8 || (K % 8) != 0 || (lda % 8) != 0) return -133;
  if (w_transposed && (swiglu || (N % 8) != 0)) return -133;
  const long long Nw = swiglu ? 2LL * N : N;
  TmapArray ta;
  CUtensorMap tb;
  for (int i = 0; i < 8; ++i) {
    const void* base = reinterpret_cast<const void*>(a_bases[i < n_bufs ? i : 0]);
    if (trlb_host::make_tmap_2d_bf16(&ta.m[i], base, (uint64_t)a_rows, (uint64_t)K, (uint64_t)lda, GBM, GBK)) return -134;
  }
  if (w_transposed ? trlb_host::make_tmap_3d_bf16(&tb, W, (uint64_t)N, (uint64_t)K, (uint64_t)E_local, (uint64_t)N,
                                                  (uint64_t)N * K, 64, GBK, 1)
                   : trlb_host::make_tmap_3d_bf16(&tb, W, (uint64_t)K, (uint64_t)Nw, (uint64_t)E_local, (uint64_t)K,
                                                  (uint64_t)Nw * K, GBK, 128, 1))
    return -135;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G_SMEM);
    attr_set = true;
  }
  GroupedParams p = {};
  p.E = n_seg; p.n_seg = n_seg; p.N = N; p.K = K; p.swiglu = swiglu; p.b_mn = w_transposed ? 1 : 0;
  p.n_tiles = swiglu ? (N + 127) / 128 : (N + GBN - 1) / GBN;
  p.k_blocks = (K + GBK - 1) / GBK;
  p.ldc = ldc; p.status = status;
  p.seg_rows = seg_rows; p.seg_a_src = seg_a_src; p.seg_a_row = seg_a_row;
  p.seg_c_dst = seg_c_dst; p.seg_c_row = seg_c_row; p.seg_w = seg_w;
  for (int i = 0; i < 8; ++i) p.c_dst[i] = reinterpret_cast<__nv_bfloat16*>(c_bases[i < n_bufs ? i : 0]);
  long long max_items = ((max_rows + GBM - 1) / GBM + n_seg) * p.n_tiles;
  int grid = trlb_host::sm_count();
  if (max_items < grid) grid = (int)max_items;
  grouped_gemm_kernel<<<grid, G_THREADS, G_SMEM, st>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

// dW[e] = G[offsets[e] : offsets[e+1]]^T . X[offsets[e] : offsets[e+1]] for every expert.  G [rows, Nw] (row stride ldg),
// X [rows, Kw] (row stride ldx), dW [E, Nw, Kw] contiguous bf16.  Nw, Kw, ldg, ldx multiples of 8.
TRLB_API int trlb_grouped_wgrad_bf16(const void* G, const void* X, const int* offsets, void* dW, long long rows, int E,
                                     int Nw, int Kw, long long ldg, long long ldx, int* status, cudaStream_t st) {
  if (E <= 0 || Nw <= 0 || Kw <= 0) return 0;
  if ((Nw % 8) != 0 || (Kw % 8) != 0 || (ldg % 8) != 0 || (ldx % 8) != 0) return -136;
  if (rows <= 0) return (int)cudaMemsetAsync(dW, 0, (size_t)E * Nw * Kw * 2, st);
  CUtensorMap tg, tx;
  // a [rows, cols] matrix read in [64 rows x 64 columns] boxes: rows are the reduction dimension
  if (trlb_host::make_tmap_2d_bf16(&tg, G, (uint64_t)rows, (uint64_t)Nw, (uint64_t)ldg, GBK, 64)) return -137;
  if (trlb_host::make_tmap_2d_bf16(&tx, X, (uint64_t)rows, (uint64_t)Kw, (uint64_t)ldx, GBK, 64)) return -138;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(grouped_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G_SMEM);
    attr_set = true;
  }
  GroupedWgradParams p = {};
  p.E = E; p.Nw = Nw; p.Kw = Kw;
  p.m_tiles = (Nw + GBM - 1) / GBM;
  p.n_tiles = (Kw + GBN - 1) / GBN;
  p.offsets = offsets; p.dW = (__nv_bfloat16*)dW; p.status = status;
  const long long items = (long long)E * p.m_tiles * p.n_tiles;
  int grid = trlb_host::sm_count();
  if (items < grid) grid = (int)items;
  grouped_wgrad_kernel<<<grid, G_THREADS, G_SMEM, st>>>(tg, tx, p);
  return (int)cudaGetLastError();
}
