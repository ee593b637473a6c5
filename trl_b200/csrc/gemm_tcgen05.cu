// Persistent warp-specialised bf16 GEMM on 5th-gen tensor cores (sm_100a):
//
//     acc[M,N] = A[M,K] . B[N,K]^T        (both operands K-major: y = x W^T of nn.Linear)
//
// * one CTA per SM, 192 threads: warp 0 = TMA producer, warp 1 = tcgen05.mma issuer,
//   warps 2-5 = epilogue (each owns one 32-lane quarter of TMEM);
// * A/B tiles (128x64 and 256x64 bf16, 128-byte swizzle) arrive through a 4-stage TMA
//   ring; accumulators (128x256 fp32) are double-buffered in TMEM (2 x 256 columns) so the
//   epilogue of tile i overlaps the MMAs of tile i+1;
// * three epilogues share the main loop:
//     EPI_STORE  C = bf16(acc + bias)
//     EPI_LSE    vocabulary-chunked online log-sum-exp for the fused lm_head: per row running
//                max / sum-exp / sum(z e^z) / label logit / argmax, never writing logits
//     EPI_DZ     d(logits) = g * (1[label] - softmax) / T written as bf16 (lm_head backward)
//
// Replaces: cuBLAS GEMM + eager softmax of trl/trainer/utils.py:1291-1424 and the chunked
// cross-entropy of trl/trainer/sft_trainer.py:117-234.
#include "common.cuh"

namespace trlb {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr size_t GEMM_SMEM = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

enum { EPI_STORE = 0, EPI_LSE = 1, EPI_DZ = 2 };

struct GemmParams {
  int M, N, K;
  // operand layouts: 0 = K-major (row-major [rows, K]: y = x W^T), 1 = MN-major (row-major [K, rows]: the operand
  // is given transposed, as dY and X are for the weight gradient and W is for the input gradient)
  int a_mn, b_mn;
  int m_tiles, n_tiles, k_blocks;
  int n_splits, tiles_per_split;  // work item = (m_tile, split); a split covers tiles_per_split N tiles
  // EPI_STORE
  __nv_bfloat16* C;
  long long ldc;
  const __nv_bfloat16* bias;
  // EPI_LSE / EPI_DZ
  const long long* labels;  // [M], may hold negative (ignored) entries
  float inv_temp;
  float4* part_stats;  // [n_splits, M]: (max2, sumexp, sum z*e^z, label logit)
  int* part_arg;       // [n_splits, M]: argmax column
  const float* lse;    // [M]  (EPI_DZ)
  const float* grow;   // [M]  dL/dlogp per row (EPI_DZ)
  const float* ent;    // [M]  entropy per row and
  const float* gent;   // [M]  dL/dentropy per row (EPI_DZ, both null when the entropy carries no gradient)
  int* status;
  // ---- all-gather fused into the GEMM (EPI_STORE only; ag_world == 0 disables) ----
  // B (the weight) lives at element offset ag_w_off of a bf16 buffer of ag_total elements that every rank
  // maps; rank r owns elements [r*ag_per, (r+1)*ag_per).  CTAs >= gemm_ctas are copiers: they pull the
  // remote parts into the local buffer, the weight's 256-row tiles first (arrival counted per tile in
  // ag_count), then the rest of the buffer.  GEMM CTAs visit N tiles starting at the first locally owned
  // one and wait (bounded) on ag_count[tile] >= ag_target before the TMA load of a tile with remote rows.
  int ag_world, ag_rank, gemm_ctas, ag_first_tile;
  long long ag_per, ag_w_off, ag_total;
  uint32_t* ag_count;
  uint32_t ag_target;
  uint32_t* ag_rest_ctr;   // dynamic chunk counter for the rest of the buffer
  uint32_t ag_rest_base;   // counter value at which this call's chunk 0 starts
  const __nv_bfloat16* ag_peer[8];
  __nv_bfloat16* ag_local;
};

__device__ __forceinline__ int ag_tile(const GemmParams& p, int nt) {
  return p.ag_world ? (nt + p.ag_first_tile) % p.n_tiles : nt;
}

__device__ __forceinline__ void item_to_coords(const GemmParams& p, int item, int& m_tile, int& n_begin, int& n_end) {
  m_tile = item % p.m_tiles;
  int split = item / p.m_tiles;
  n_begin = split * p.tiles_per_split;
  n_end = min(n_begin + p.tiles_per_split, p.n_tiles);
}

__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// element range [e0, e1) of the shared buffer covered by weight tile nt
__device__ __forceinline__ void ag_tile_range(const GemmParams& p, int nt, long long& e0, long long& e1) {
  e0 = p.ag_w_off + (long long)nt * BN * p.K;
  const long long end = p.ag_w_off + (long long)p.N * p.K;
  e1 = e0 + (long long)BN * p.K;
  if (e1 > end) e1 = end;
}
__device__ __forceinline__ bool ag_tile_is_local(const GemmParams& p, int nt) {
  long long e0, e1;
  ag_tile_range(p, nt, e0, e1);
  return e0 / p.ag_per == p.ag_rank && (e1 - 1) / p.ag_per == p.ag_rank;
}

// ---- copier CTAs: peer -> shared memory -> local global memory with bulk async copies ----------------
// One thread drives a ring of COPY_STAGES x COPY_CHUNK bytes in the (otherwise unused) tile ring of this CTA:
// cp.async.bulk loads from the owner's memory complete on an mbarrier, cp.async.bulk stores write the local
// buffer.  About 160 KB are in flight per copier CTA, which is what NVLink latency needs; no registers or
// warps are spent on the data.  Weight tiles are signalled (arrival counter per tile) once the bulk group
// holding their last chunk has completed.
constexpr int COPY_STAGES = 6;
constexpr uint32_t COPY_CHUNK = 32768;

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}

struct CopyRing {
  uint8_t* smem;
  uint64_t* bars;
  int issued = 0;     // loads issued
  int stored = 0;     // stores issued (= bulk groups committed)
  // pending loads (ring order)
  __nv_bfloat16* dst[COPY_STAGES];
  uint32_t bytes[COPY_STAGES];
  int tile_of[COPY_STAGES];  // weight tile to signal after this chunk's store, or -1
};

// Signals are delayed until the store's bulk group has completed: group g is known complete once
// wait_group<k> ran after committing group g + k.
struct PendingSignal { int group, tile; };

__device__ bool ag_copy_stream(const GemmParams& p, CopyRing& R, PendingSignal* sig, int& n_sig, long long e0,
                               long long e1, int tile, volatile int* abort_flag) {
  // splits [e0, e1) into chunks that do not cross an owner boundary; own data is skipped
  long long e = e0;
  while (true) {
    const bool more = e < e1;
    // keep COPY_STAGES - 2 loads in flight; drain when there is nothing more to issue
    if (more && R.issued - R.stored < COPY_STAGES - 1) {
      const int owner = (int)(e / p.ag_per);
      long long lim = min(e1, (long long)(owner + 1) * p.ag_per);
      long long n = min(lim - e, (long long)(COPY_CHUNK / 2));
      if (owner != p.ag_rank) {
        const int s = R.issued % COPY_STAGES;
        // stage s was used by chunk issued - COPY_STAGES: its store (group issued - COPY_STAGES) must have
        // finished reading shared memory; at most 2 groups are younger than it
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        mbar_expect_tx(&R.bars[s], (uint32_t)(n * 2));
        bulk_load(R.smem + (size_t)s * COPY_CHUNK, p.ag_peer[owner] + e, (uint32_t)(n * 2), &R.bars[s]);
        R.dst[s] = p.ag_local + e;
        R.bytes[s] = (uint32_t)(n * 2);
        R.tile_of[s] = (e + n >= e1) ? tile : -1;
        ++R.issued;
      } else if (e + n >= e1 && tile >= 0) {
        // the tail of this tile slice is local data: signal after everything issued so far has landed
        sig[n_sig++] = PendingSignal{R.issued - 1, tile};
      }
      e += n;
      continue;
    }
    if (!more) return true;  // loads may stay in flight: the next range (or ag_drain) continues the ring
    {
      const int s = R.stored % COPY_STAGES;
      if (!mbar_wait(&R.bars[s], (uint32_t)((R.stored / COPY_STAGES) & 1), abort_flag, p.status, 160)) return false;
      bulk_store(R.dst[s], R.smem + (size_t)s * COPY_CHUNK, R.bytes[s]);
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      if (R.tile_of[s] >= 0) sig[n_sig++] = PendingSignal{R.stored, R.tile_of[s]};
      ++R.stored;
      asm volatile("cp.async.bulk.wait_group 2;" ::: "memory");  // groups <= stored - 3 are complete
      int k = 0;
      for (int i = 0; i < n_sig; ++i) {
        if (sig[i].group <= R.stored - 3) {
          asm volatile("fence.proxy.async.global;" ::: "memory");
          __threadfence();
          atomicAdd(p.ag_count + sig[i].tile, 1u);
        } else {
          sig[k++] = sig[i];
        }
      }
      n_sig = k;
    }
  }
  return true;
}

// Store every pending load, wait for all stores, publish the remaining tile arrivals.
__device__ void ag_drain(const GemmParams& p, CopyRing& R, PendingSignal* sig, int& n_sig, volatile int* abort_flag,
                         bool ok) {
  while (ok && R.stored < R.issued) {
    const int s = R.stored % COPY_STAGES;
    if (!mbar_wait(&R.bars[s], (uint32_t)((R.stored / COPY_STAGES) & 1), abort_flag, p.status, 161)) { ok = false; break; }
    bulk_store(R.dst[s], R.smem + (size_t)s * COPY_CHUNK, R.bytes[s]);
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    if (R.tile_of[s] >= 0) sig[n_sig++] = PendingSignal{R.stored, R.tile_of[s]};
    ++R.stored;
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  asm volatile("fence.proxy.async.global;" ::: "memory");
  __threadfence();
  for (int i = 0; i < n_sig; ++i) atomicAdd(p.ag_count + sig[i].tile, 1u);
  n_sig = 0;
}

// The rest of the buffer (the layer's other weights) is cut into 256 KB work items handed out by an atomic
// counter, so dedicated copiers and GEMM CTAs that have run out of tiles share it evenly.
constexpr long long REST_ITEM = 131072;  // elements

__device__ bool ag_help_rest(const GemmParams& p, CopyRing& R, PendingSignal* sig, int& n_sig, volatile int* abort_flag) {
  const long long w_end = p.ag_w_off + (long long)p.N * p.K;
  const long long n_a = (p.ag_w_off + REST_ITEM - 1) / REST_ITEM, n_b = (p.ag_total - w_end + REST_ITEM - 1) / REST_ITEM;
  while (true) {
    const long long id = (long long)(atomicAdd(p.ag_rest_ctr, 1u) - p.ag_rest_base);
    if (id >= n_a + n_b) return true;
    long long e0, e1;
    if (id < n_a) { e0 = id * REST_ITEM; e1 = min(p.ag_w_off, e0 + REST_ITEM); }
    else { e0 = w_end + (id - n_a) * REST_ITEM; e1 = min(p.ag_total, e0 + REST_ITEM); }
    if (!ag_copy_stream(p, R, sig, n_sig, e0, e1, -1, abort_flag)) return false;
  }
}

__device__ void ag_copier(const GemmParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag) {
  if (threadIdx.x != 0) return;
  const int part = (int)blockIdx.x, parts = (int)gridDim.x - p.gemm_ctas;
  CopyRing R;
  R.smem = smem;
  R.bars = bars;
  PendingSignal sig[16];
  int n_sig = 0;
  bool ok = true;
  for (int i = 0; i < p.n_tiles && ok; ++i) {
    const int nt = ag_tile(p, i);
    if (ag_tile_is_local(p, nt)) continue;
    long long e0, e1;
    ag_tile_range(p, nt, e0, e1);
    const long long nvec = (e1 - e0) / 8, per_part = (nvec + parts - 1) / parts;
    const long long v0 = min(nvec, part * per_part), v1 = min(nvec, v0 + per_part);
    if (v1 > v0) ok = ag_copy_stream(p, R, sig, n_sig, e0 + v0 * 8, e0 + v1 * 8, nt, abort_flag);
    else sig[n_sig++] = PendingSignal{R.issued - 1, nt};  // empty slice: still counts as an arrival
  }
  if (ok) ok = ag_help_rest(p, R, sig, n_sig, abort_flag);
  ag_drain(p, R, sig, n_sig, abort_flag, ok);
}

template <int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                 // [STAGES]
  uint64_t* empty_bar = bars + STAGES;       // [STAGES]
  uint64_t* tfull_bar = bars + 2 * STAGES;   // [2]
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_items = p.m_tiles * p.n_splits;
  // copier CTAs take the lowest block indices so that they are scheduled first
  const int n_cop = p.ag_world > 0 ? (int)gridDim.x - p.gemm_ctas : 0;
  const bool copier = (int)blockIdx.x < n_cop;
  const int item_stride = p.ag_world > 0 ? p.gemm_ctas : (int)gridDim.x;
  const int first_item = copier ? total_items : (int)blockIdx.x - n_cop;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (copier) {
    ag_copier(p, tiles, bars, abort_flag);
  } else if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = first_item; item < total_items && ok; item += item_stride) {
        int m_tile, n0, n1;
        item_to_coords(p, item, m_tile, n0, n1);
        for (int nt = n0; nt < n1 && ok; ++nt) {
          const int nta = ag_tile(p, nt);
          if (p.ag_world > 0 && !ag_tile_is_local(p, nta)) {
            // rows of this tile come from peers: wait until every copier has delivered its slice
            const uint64_t t0 = globaltimer_ns();
            while ((int32_t)(ld_acquire_gpu_u32(p.ag_count + nta) - p.ag_target) < 0) {
              if (*abort_flag) { ok = false; break; }
              if (globaltimer_ns() - t0 > kWaitBudgetNs) {
                *abort_flag = 1;
                report_error(p.status, ERR_WAIT_TIMEOUT, 150, nta);
                ok = false;
                break;
              }
              __nanosleep(32);
            }
            if (!ok) break;
            asm volatile("fence.proxy.async.global;" ::: "memory");  // copier stores (generic proxy) -> TMA reads
          }
          for (int kb = 0; kb < p.k_blocks; ++kb) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 100 + stage)) { ok = false; break; }
            uint8_t* sa = tiles + stage * STAGE_BYTES;
            uint8_t* sb = sa + A_BYTES;
            mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
            if (p.a_mn) {  // [64 k-rows x 64] boxes, one per 64 rows of the tile
#pragma unroll
              for (int b = 0; b < BM / 64; ++b)
                tma_load_2d(sa + b * 8192, &tmap_a, &full_bar[stage], m_tile * BM + b * 64, kb * BK);
            } else {
              tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * BK, m_tile * BM);
            }
            if (p.b_mn) {
#pragma unroll
              for (int b = 0; b < BN / 64; ++b)
                tma_load_2d(sb + b * 8192, &tmap_b, &full_bar[stage], nta * BN + b * 64, kb * BK);
            } else {
              tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * BK, nta * BN);
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16_major(BM, BN, p.a_mn != 0, p.b_mn != 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int item = first_item; item < total_items && ok; item += item_stride) {
        int m_tile, n0, n1;
        item_to_coords(p, item, m_tile, n0, n1);
        for (int nt = n0; nt < n1 && ok; ++nt) {
          if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, 200 + acc)) { ok = false; break; }
          tc_fence_after();
          const uint32_t tacc = tmem_base + (uint32_t)acc * BN;
          for (int kb = 0; kb < p.k_blocks; ++kb) {
            if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 300 + stage)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_u32(tiles + stage * STAGE_BYTES);
            // K-major: a K step of 16 bf16 is 32 bytes inside the swizzle atom (2 address units);
            // MN-major: 16 k-rows of 128 bytes (2048 bytes = 128 address units), 64-element groups 8 KB apart
            const uint64_t adesc = p.a_mn ? umma_desc_mnmajor_sw128(sa, 8192) : umma_desc_kmajor_sw128(sa);
            const uint64_t bdesc = p.b_mn ? umma_desc_mnmajor_sw128(sa + A_BYTES, 8192) : umma_desc_kmajor_sw128(sa + A_BYTES);
            const uint32_t astep = p.a_mn ? 128u : 2u, bstep = p.b_mn ? 128u : 2u;
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk)
              umma_bf16_ss(tacc, adesc + astep * kk, bdesc + bstep * kk, idesc, (kb | kk) != 0);
            umma_commit(&empty_bar[stage]);  // smem stage reusable once these MMAs retire
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          umma_commit(&tfull_bar[acc]);  // accumulator complete
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue warps (2..5) ----------------
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32)
    const int row_in_tile = quarter * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    constexpr float LOG2E = 1.4426950408889634f;
    for (int item = first_item; item < total_items && ok; item += item_stride) {
      int m_tile, n0, n1;
      item_to_coords(p, item, m_tile, n0, n1);
      const int row = m_tile * BM + row_in_tile;
      const bool row_ok = row < p.M;
      // per-row running statistics (EPI_LSE)
      float run_max = -INFINITY, run_sum = 0.f, run_zsum = 0.f, tgt = 0.f;
      int arg = 0;
      long long label = -1;
      float lse_row = 0.f, g_row = 0.f, ent_row = 0.f, gent_row = 0.f;
      if (EPI != EPI_STORE && row_ok) {
        label = p.labels[row];
        if (EPI == EPI_DZ) {
          lse_row = p.lse[row];
          g_row = p.grow[row];
          if (p.gent != nullptr) { ent_row = p.ent[row]; gent_row = p.gent[row]; }
        }
      }
      for (int nt = n0; nt < n1 && ok; ++nt) {
        if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, 400 + acc)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tacc = tmem_base + (uint32_t)acc * BN + ((uint32_t)(quarter * 32) << 16);
        const int col0 = ag_tile(p, nt) * BN;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          float v[32];
          tmem_ld_32x32(tacc + c, v);
          tmem_ld_wait();
          const int cbase = col0 + c;
          if (EPI == EPI_STORE) {
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
          } else if (EPI == EPI_LSE) {
            if (cbase < p.N) {
              const float sc = p.inv_temp;
              float cmax = -INFINITY;
              const int rel = (int)(label - cbase);
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                float z = (cbase + i < p.N) ? v[i] * sc : -INFINITY;
                v[i] = z;
                if (z > cmax) cmax = z;
                if (i == rel) tgt = z;
              }
              if (cmax > run_max) {
                // first column reaching the new maximum (ties: lowest index, like torch.argmax)
                int a = 0;
#pragma unroll
                for (int i = 31; i >= 0; --i)
                  if (v[i] == cmax) a = i;
                arg = cbase + a;
                const float scale = exp2f((run_max - cmax) * LOG2E);
                run_sum *= scale;
                run_zsum *= scale;
                run_max = cmax;
              }
              const float mb = run_max * LOG2E;
              float s = 0.f, zs = 0.f;
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float e = exp2f(fmaf(v[i], LOG2E, -mb));
                s += e;
                zs = fmaf(e, (cbase + i < p.N) ? v[i] : 0.f, zs);
              }
              run_sum += s;
              run_zsum += zs;
            }
          } else {  // EPI_DZ
            if (row_ok && cbase < p.N) {
              __nv_bfloat16* dst = p.C + (long long)row * p.ldc + cbase;
              const float sc = p.inv_temp;
              const float gs = g_row * sc, ge = gent_row * sc;
              const int rel = (int)(label - cbase);
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                // d logp_label / dz_j = (1[j = label] - p_j) / T;  dH / dz_j = -p_j (log p_j + H) / T
                const float lp = fmaf(v[i], sc, -lse_row);
                const float pr = __expf(lp);
                v[i] = gs * ((i == rel ? 1.f : 0.f) - pr) - ge * pr * (lp + ent_row);
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
        }
        // release this accumulator to the MMA warp
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (EPI == EPI_LSE && ok && row_ok) {
        const int split = item / p.m_tiles;
        p.part_stats[(long long)split * p.M + row] = make_float4(run_max, run_sum, run_zsum, tgt);
        p.part_arg[(long long)split * p.M + row] = arg;
      }
    }
  }

  // ---------------- teardown (also the abort path) ----------------
  __syncthreads();
  if (p.ag_world > 0 && !copier && !*abort_flag) {
    // this CTA has no tiles left: its tile ring becomes a copy ring and it joins the gather
    if (threadIdx.x == 0) {
      for (int s = 0; s < COPY_STAGES; ++s) {
        asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(&bars[s])) : "memory");
        mbar_init(&bars[s], 1);
      }
      mbar_fence_init();
      CopyRing R;
      R.smem = tiles;
      R.bars = bars;
      PendingSignal sig[16];
      int n_sig = 0;
      const bool ok = ag_help_rest(p, R, sig, n_sig, abort_flag);
      ag_drain(p, R, sig, n_sig, abort_flag, ok);
    }
    __syncthreads();
  }
  if (*abort_flag) {
    // give TMA copies that may still be in flight time to land before shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Combine per-split statistics into log p(label), entropy, log-sum-exp and argmax.
__global__ void lse_combine_kernel(const float4* __restrict__ part, const int* __restrict__ part_arg, int n_splits, int M,
                                   float* __restrict__ logp, float* __restrict__ entropy, float* __restrict__ lse_out,
                                   int* __restrict__ argmax_out) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  float mx = -INFINITY;
  int arg = 0;
  for (int s = 0; s < n_splits; ++s) {
    const float m = part[(long long)s * M + row].x;
    if (m > mx) { mx = m; arg = part_arg[(long long)s * M + row]; }
  }
  float sum = 0.f, zsum = 0.f, tgt = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float4 q = part[(long long)s * M + row];
    const float sc = __expf(q.x - mx);
    sum += q.y * sc;
    zsum += q.z * sc;
    tgt += q.w;  // exactly one split holds the label column, the others contribute 0
  }
  const float lse = mx + __logf(sum);
  if (logp) logp[row] = tgt - lse;
  if (entropy) entropy[row] = lse - zsum / sum;
  if (lse_out) lse_out[row] = lse;
  if (argmax_out) argmax_out[row] = arg;
}

}  // namespace trlb

// ------------------------------------------------------------------------------------------------
// host launchers (C ABI)
// ------------------------------------------------------------------------------------------------
using namespace trlb;

template <int EPI>
static int launch_gemm(const void* A, const void* B, GemmParams p, long long lda, long long ldb, cudaStream_t stream) {
  if (p.M <= 0 || p.N <= 0 || p.K <= 0) return 0;
  if ((lda % 8) != 0 || (ldb % 8) != 0) return -100;  // 16-byte TMA stride rule
  if ((!p.a_mn || !p.b_mn) && (p.K % 8) != 0) return -100;
  CUtensorMap ta, tb;
  // a K-major operand is a [rows, K] matrix read in [tile rows x 64] boxes; an MN-major one is a [K, rows] matrix read
  // in [64 x 64] boxes (64 k-rows of 64 contiguous operand rows)
  int r = p.a_mn ? trlb_host::make_tmap_2d_bf16(&ta, A, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)lda, BK, 64)
                 : trlb_host::make_tmap_2d_bf16(&ta, A, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)lda, BM, BK);
  if (r) return -101;
  r = p.b_mn ? trlb_host::make_tmap_2d_bf16(&tb, B, (uint64_t)p.K, (uint64_t)p.N, (uint64_t)ldb, BK, 64)
             : trlb_host::make_tmap_2d_bf16(&tb, B, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)ldb, BN, BK);
  if (r) return -102;
  p.m_tiles = (p.M + BM - 1) / BM;
  p.n_tiles = (p.N + BN - 1) / BN;
  p.k_blocks = (p.K + BK - 1) / BK;
  if (EPI == EPI_STORE || EPI == EPI_DZ) {
    p.n_splits = p.n_tiles;
    p.tiles_per_split = 1;
  } else {
    p.tiles_per_split = (p.n_tiles + p.n_splits - 1) / p.n_splits;
  }
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemm_tn_kernel<EPI_STORE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM);
    cudaFuncSetAttribute(gemm_tn_kernel<EPI_LSE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM);
    cudaFuncSetAttribute(gemm_tn_kernel<EPI_DZ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM);
    attr_set = true;
  }
  const int items = p.m_tiles * p.n_splits;
  int grid = items < trlb_host::sm_count() ? items : trlb_host::sm_count();
  if (p.ag_world > 0) {
    const int copiers = p.gemm_ctas;  // the caller passed the copier count here
    int workers = trlb_host::sm_count() - copiers;
    if (workers > items) workers = items;
    if (workers < 1) return -103;
    p.gemm_ctas = workers;
    grid = workers + copiers;
  }
  gemm_tn_kernel<EPI><<<grid, GEMM_THREADS, GEMM_SMEM, stream>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

// C[M,N] (bf16, row stride ldc) = A[M,K] . B[N,K]^T (+ bias[N])
TRLB_API int trlb_gemm_bf16_tn(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                               long long lda, long long ldb, long long ldc, int* status, cudaStream_t stream) {
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.C = (__nv_bfloat16*)C; p.ldc = ldc; p.bias = (const __nv_bfloat16*)bias;
  p.status = status;
  return launch_gemm<EPI_STORE>(A, B, p, lda, ldb, stream);
}

// General form: C[M,N] (bf16) = op(A) . op(B)^T (+ bias[N]) with each operand either K-major ([rows, K] row-major,
// a_mn / b_mn = 0) or MN-major ([K, rows] row-major, = 1).  With x [T, K], W [N, K], dY [T, N]:
//   forward   Y  = x W^T      A = x  (K-major),  B = W  (K-major)
//   dgrad     dX = dY W       A = dY (K-major),  B = W  (MN-major: [N = contraction, K = output columns])
//   wgrad     dW = dY^T x     A = dY (MN-major: [T = contraction, N = output rows]),  B = x (MN-major)
// No operand is ever transposed in memory.  MN-major operands need their row count (M or N) to be a multiple of 8.
TRLB_API int trlb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long long lda,
                            long long ldb, long long ldc, int a_mn, int b_mn, int* status, cudaStream_t stream) {
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K; p.a_mn = a_mn ? 1 : 0; p.b_mn = b_mn ? 1 : 0;
  if ((p.a_mn && (M % 8)) || (p.b_mn && (N % 8))) return -100;
  p.C = (__nv_bfloat16*)C; p.ldc = ldc; p.bias = (const __nv_bfloat16*)bias;
  p.status = status;
  return launch_gemm<EPI_STORE>(A, B, p, lda, ldb, stream);
}

// Number of vocabulary splits the forward uses for M rows (so callers can size the scratch).
TRLB_API int trlb_lmhead_num_splits(int M, int V) {
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (V + BN - 1) / BN;
  const int sms = trlb_host::sm_count();
  int splits = (2 * sms + m_tiles - 1) / m_tiles;
  if (splits < 1) splits = 1;
  if (splits > n_tiles) splits = n_tiles;
  if (splits > 64) splits = 64;
  // normalise so that no split is empty
  const int tps = (n_tiles + splits - 1) / splits;
  return (n_tiles + tps - 1) / tps;
}

// Fused lm_head forward.  H[M,K] bf16, W[V,K] bf16, labels[M] int64.
// scratch: part_stats float4[n_splits*M], part_arg int[n_splits*M] with n_splits = trlb_lmhead_num_splits(M,V).
// Outputs (each may be null): logp[M], entropy[M], lse[M] fp32, argmax[M] int32.
TRLB_API int trlb_lmhead_fwd(const void* H, const void* W, const long long* labels, int M, int V, int K, long long ldh,
                             long long ldw, float inv_temp, void* part_stats, int* part_arg, int n_splits, float* logp,
                             float* entropy, float* lse, int* argmax, int* status, cudaStream_t stream) {
  GemmParams p = {};
  p.M = M; p.N = V; p.K = K;
  p.labels = labels; p.inv_temp = inv_temp;
  p.part_stats = (float4*)part_stats; p.part_arg = part_arg;
  p.n_splits = n_splits;
  p.status = status;
  int r = launch_gemm<EPI_LSE>(H, W, p, ldh, ldw, stream);
  if (r) return r;
  lse_combine_kernel<<<(M + 255) / 256, 256, 0, stream>>>((const float4*)part_stats, part_arg, n_splits, M, logp, entropy,
                                                         lse, argmax);
  return (int)cudaGetLastError();
}

// Fused lm_head backward, stage 1: dZ[M,V] (bf16, row stride ldz) = grow * (1[label] - softmax(z/T)) / T
// and, when gent is given, - gent * p * (log p + ent) / T (the gradient of the row's entropy); ent / gent may be null.
TRLB_API int trlb_lmhead_dz(const void* H, const void* W, const long long* labels, const float* lse, const float* grow,
                            const float* ent, const float* gent, void* dZ, int M, int V, int K, long long ldh,
                            long long ldw, long long ldz, float inv_temp, int* status, cudaStream_t stream) {
  GemmParams p = {};
  p.M = M; p.N = V; p.K = K;
  p.labels = labels; p.inv_temp = inv_temp; p.lse = lse; p.grow = grow;
  p.ent = gent != nullptr ? ent : nullptr; p.gent = ent != nullptr ? gent : nullptr;
  p.C = (__nv_bfloat16*)dZ; p.ldc = ldz;
  p.status = status;
  return launch_gemm<EPI_DZ>(H, W, p, ldh, ldw, stream);
}

// All-gather fused into the GEMM: C[M,N] = A[M,K] . W[N,K]^T where W sits at element offset w_off of a bf16
// buffer of `total` elements that every rank maps (peers[r] = rank r's address of the buffer, peers[rank] is
// local) and rank r holds valid data only for elements [r*per, (r+1)*per).  On return (stream order) the
// whole local buffer is complete.  ag_count: zero-initialised uint32 per N tile (256 rows), reused across
// calls with a target that grows by `copiers` per call (pass the call number in `call_index`, from 1).
TRLB_API int trlb_ag_gemm_bf16_tn(const void* A, void* C, const void* bias, int M, int N, int K, long long lda,
                                  long long ldc, const unsigned long long* peers, int rank, int world, long long per,
                                  long long w_off, long long total, unsigned* ag_count, int call_index, int copiers,
                                  int* status, cudaStream_t stream) {
  if (world < 1 || world > 8 || per % 8 != 0 || w_off % 8 != 0 || total % 8 != 0 || (long long)N * K % 8 != 0) return -110;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.C = (__nv_bfloat16*)C; p.ldc = ldc; p.bias = (const __nv_bfloat16*)bias;
  p.status = status;
  p.ag_world = world; p.ag_rank = rank; p.ag_per = per; p.ag_w_off = w_off; p.ag_total = total;
  p.ag_count = ag_count; p.ag_target = (unsigned)call_index * (unsigned)copiers;
  // the last word of the counter array hands out rest-of-buffer work items; zeroed (stream order) per call
  p.ag_rest_ctr = ag_count + 4095;
  p.ag_rest_base = 0;
  if ((N + BN - 1) / BN > 4095) return -111;
  if (cudaMemsetAsync(p.ag_rest_ctr, 0, sizeof(unsigned), stream) != cudaSuccess) return -112;
  for (int i = 0; i < 8; ++i) p.ag_peer[i] = i < world ? reinterpret_cast<const __nv_bfloat16*>(peers[i]) : nullptr;
  p.ag_local = reinterpret_cast<__nv_bfloat16*>(peers[rank]);
  p.gemm_ctas = copiers;
  // first locally owned tile of W (or tile 0 when this rank owns none of W)
  const long long own0 = (long long)rank * per, own1 = own0 + per, wend = w_off + (long long)N * K;
  long long first = 0;
  if (own1 > w_off && own0 < wend) {
    const long long s = own0 > w_off ? own0 - w_off : 0;
    first = (s + (long long)BN * K - 1) / ((long long)BN * K);
  }
  const int n_tiles = (N + BN - 1) / BN;
  p.ag_first_tile = (int)(first % n_tiles);
  const void* B = reinterpret_cast<const __nv_bfloat16*>(peers[rank]) + w_off;
  return launch_gemm<EPI_STORE>(A, B, p, lda, (long long)K, stream);
}
