// Paged decode attention on the 5th-generation tensor cores (one new token per sequence, grouped-query models).
//
// Cache layout this kernel reads (head_dim 128, 64-token pages):
//   K   [num_blocks, 64 tokens, Hk, 128]      a page of one head is 64 rows of 128 dims
//   V^T [num_blocks, Hk, 128 dims, 64 tokens] V is stored transposed inside a page, so both operands of both
//                                             products are K-major tiles that TMA delivers in the 128-byte swizzle
// Work item = (sequence, KV head, split of the KV range).  Per 128-token tile:
//   S^T[128 tok, 16]  = K_tile[128 tok, 128 dims] . Q^T      (Q: the G <= 8 query heads of this KV head, zero padded)
//   P                 = exp2(S^T * scale - running max)      (softmax warps; written to shared memory as bf16)
//   O^T[128 dims, 16] = V^T_tile[128 dims, 128 tok] . P^T
// A persistent CTA per SM: warp 0 = TMA producer (3-stage ring of 64 KB K+V tiles), warp 1 = tcgen05.mma issuer
// (S^T double-buffered in TMEM so the next tile's QK^T runs under the softmax of the current one), warps 2-5 = softmax
// and output accumulation (one thread per token for S^T, one thread per head dim for O^T, running sums in registers).
// Partials (m, l, o) per split are merged by paged_attn_combine_kernel.
//
// The reference leaves this op to vLLM's paged attention (trl/generation/vllm_generation.py); nothing to port.
#include "common.cuh"
#include "decode_attn.cuh"

namespace trlb {

constexpr int TC_THREADS = 192;
constexpr int TC_STAGES = 3;
constexpr uint32_t TC_STAGE_BYTES = 65536;   // K: 2 d-halves x [128 tok x 64 dims]; V^T: 2 pages x [128 dims x 64 tok]
constexpr uint32_t TC_Q_BYTES = 4096;        // 2 d-halves x [16 rows x 64 dims]
constexpr uint32_t TC_P_BYTES = 4096;        // 2 pages x [16 rows x 64 tok]
constexpr uint32_t TC_TMEM_COLS = 64;        // S0 [0,16) S1 [16,32) O [32,48)
constexpr size_t TC_SMEM = TC_STAGES * TC_STAGE_BYTES + 2 * TC_Q_BYTES + TC_P_BYTES + 1024 /*barriers, reductions*/ +
                           1024 /*alignment slack*/;

struct TcAttnParams {
  const __nv_bfloat16* q;  // [B, Hq, 128]
  const int* seq_lens;
  const int* slot_ids;
  const int* block_table;
  int max_blocks, B, Hq, Hk, splits;
  float scale_log2;
  float* part_o;   // [B, Hq, splits, 128]
  float* part_ml;  // [B, Hq, splits, 2]
  __nv_bfloat16* out;  // [B, Hq, 128]; written directly (normalised) when splits == 1, else by the combine kernel
  int* status;
};

__device__ __forceinline__ bool bar_and_128(bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"((uint32_t)pred)
      : "memory");
  return out != 0;
}

struct TcItem {
  int b, kvh, sp, slot, len, t0, t1;
};

__device__ __forceinline__ TcItem tc_item(const TcAttnParams& p, int item) {
  TcItem it;
  const int per = p.B * p.Hk;
  it.sp = item / per;
  const int rem = item % per;
  it.kvh = rem / p.B;
  it.b = rem % p.B;
  it.slot = p.slot_ids ? p.slot_ids[it.b] : it.b;
  const int sl = p.seq_lens[it.slot];
  it.len = sl < 0 ? 0 : sl + 1;  // the new token was appended before attention; negative = inactive slot
  const int n_t = (it.len + 127) >> 7;
  const int tps = (n_t + p.splits - 1) / p.splits;
  it.t0 = min(n_t, it.sp * tps);
  it.t1 = min(n_t, it.t0 + tps);
  return it;
}

__global__ void __launch_bounds__(TC_THREADS, 1)
paged_decode_attn_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                            const TcAttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  uint8_t* q_s = smem + TC_STAGES * TC_STAGE_BYTES;  // two buffers
  uint8_t* p_s = q_s + 2 * TC_Q_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + TC_P_BYTES);
  uint64_t* full_bar = bars;                    // [3]
  uint64_t* empty_bar = bars + TC_STAGES;       // [3]
  uint64_t* sfull_bar = bars + 2 * TC_STAGES;   // [2]
  uint64_t* pfull_bar = sfull_bar + 2;          // [1]
  uint64_t* ofull_bar = pfull_bar + 1;          // [1]
  uint64_t* qfull_bar = ofull_bar + 1;          // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(qfull_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red_m = reinterpret_cast<float*>(tmem_slot + 4);  // [4][8]
  float* red_l = red_m + 32;                               // [4][8]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_items = p.B * p.Hk * p.splits;
  const int G = p.Hq / p.Hk;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&sfull_bar[0], 1);
    mbar_init(&sfull_bar[1], 1);
    mbar_init(pfull_bar, 128);
    mbar_init(ofull_bar, 1);
    mbar_init(&qfull_bar[0], 128);
    mbar_init(&qfull_bar[1], 128);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  // P rows 8..15 are never written by the softmax warps: zero the whole buffer once
  for (int i = threadIdx.x; i < (int)(TC_P_BYTES / 16); i += TC_THREADS)
    reinterpret_cast<uint4*>(p_s)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  if (warp == 1) {
    tmem_alloc(tmem_slot, TC_TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();  // after the TMEM allocation, see common.cuh
  pdl_wait();               // q and the newest K/V rows come from the kernel before this one

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int m = 0;  // tiles issued by this CTA
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const TcItem it = tc_item(p, item);
        const int n_pages = (it.len + 63) >> 6;
        const int* bt = p.block_table + (size_t)it.slot * p.max_blocks;
        for (int t = it.t0; t < it.t1; ++t, ++m) {
          const int stage = m % TC_STAGES;
          if (!mbar_wait(&empty_bar[stage], (uint32_t)(((m / TC_STAGES) & 1) ^ 1), abort_flag, p.status, 700 + stage)) {
            ok = false;
            break;
          }
          const int pg0 = 2 * t;
          const int pg1 = (pg0 + 1 < n_pages) ? pg0 + 1 : pg0;  // past the end: the same page again, its scores are masked
          const int blk0 = bt[pg0], blk1 = bt[pg1];
          uint8_t* st = stages + (size_t)stage * TC_STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], TC_STAGE_BYTES);
          for (int h = 0; h < 2; ++h) {
            tma_load_3d(st + h * 16384, &tmap_k, &full_bar[stage], h * 64, it.kvh, blk0 * 64);
            tma_load_3d(st + h * 16384 + 8192, &tmap_k, &full_bar[stage], h * 64, it.kvh, blk1 * 64);
          }
          tma_load_2d(st + 32768, &tmap_v, &full_bar[stage], 0, (blk0 * p.Hk + it.kvh) * 128);
          tma_load_2d(st + 49152, &tmap_v, &full_bar[stage], 0, (blk1 * p.Hk + it.kvh) * 128);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, 16);
      const uint32_t stages_u = smem_u32(stages), q_u = smem_u32(q_s), p_u = smem_u32(p_s);
      int m = 0, j = 0;
      bool ok = true;
      auto mma1 = [&](int mm, int jj) -> bool {
        const int stage = mm % TC_STAGES;
        if (!mbar_wait(&full_bar[stage], (uint32_t)((mm / TC_STAGES) & 1), abort_flag, p.status, 710 + stage)) return false;
        tc_fence_after();
        const uint32_t ts = tmem_base + (uint32_t)(mm & 1) * 16;
        const uint32_t kb_base = stages_u + (uint32_t)stage * TC_STAGE_BYTES, qb = q_u + (uint32_t)(jj & 1) * TC_Q_BYTES;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t adesc = umma_desc_kmajor_sw128(kb_base + kb * 16384);
          const uint64_t bdesc = umma_desc_kmajor_sw128(qb + kb * 2048);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_bf16_ss(ts, adesc + 2 * kk, bdesc + 2 * kk, idesc, (kb | kk) != 0);
        }
        umma_commit(&sfull_bar[mm & 1]);
        return true;
      };
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++j) {
        const TcItem it = tc_item(p, item);
        if (!mbar_wait(&qfull_bar[j & 1], (uint32_t)((j >> 1) & 1), abort_flag, p.status, 720)) { ok = false; break; }
        const int T = it.t1 - it.t0;
        if (T == 0) continue;
        tc_fence_after();
        if (!mma1(m, j)) { ok = false; break; }
        for (int i = 0; i < T; ++i) {
          if (i + 1 < T && !mma1(m + i + 1, j)) { ok = false; break; }
          const int mm = m + i, stage = mm % TC_STAGES;
          if (!mbar_wait(pfull_bar, (uint32_t)(mm & 1), abort_flag, p.status, 730)) { ok = false; break; }
          tc_fence_after();
          const uint32_t to = tmem_base + 32;
          const uint32_t vb = stages_u + (uint32_t)stage * TC_STAGE_BYTES + 32768;
#pragma unroll
          for (int pg = 0; pg < 2; ++pg) {
            const uint64_t adesc = umma_desc_kmajor_sw128(vb + pg * 16384);
            const uint64_t bdesc = umma_desc_kmajor_sw128(p_u + pg * 2048);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) umma_bf16_ss(to, adesc + 2 * kk, bdesc + 2 * kk, idesc, (pg | kk) != 0);
          }
          umma_commit(ofull_bar);
          umma_commit(&empty_bar[stage]);
        }
        m += T;
      }
    }
    __syncwarp();
  } else {
    // ---------------- softmax + output accumulation (128 threads) ----------------
    const int quarter = warp & 3;              // TMEM lane quarter this warp may read
    const int row = quarter * 32 + lane;       // token row of S^T, head-dim row of O^T
    const int ts = threadIdx.x - 64;           // 0..127
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    constexpr float LN2 = 0.6931471805599453f;
    bool good = true;
    int m_cnt = 0, j = 0;

    auto write_q = [&](int item, int buf) {
      const TcItem it = tc_item(p, item);
      uint8_t* dst = q_s + (size_t)buf * TC_Q_BYTES;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int ch = ts + 128 * i;          // 16 rows x 16 chunks of 8 dims
        const int r = ch >> 4, cc = ch & 15, kb = cc >> 3, c8 = cc & 7;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < G) v = *reinterpret_cast<const uint4*>(p.q + ((size_t)it.b * p.Hq + it.kvh * G + r) * 128 + cc * 8);
        *reinterpret_cast<uint4*>(dst + kb * 2048 + (r >> 3) * 1024 + (r & 7) * 128 + ((c8 ^ (r & 7)) << 4)) = v;
      }
      fence_proxy_async_smem();
      mbar_arrive(&qfull_bar[buf]);
    };

    if ((int)blockIdx.x < n_items) write_q(blockIdx.x, 0);
    for (int item = blockIdx.x; item < n_items && good; item += gridDim.x, ++j) {
      if (item + (int)gridDim.x < n_items) write_q(item + gridDim.x, (j + 1) & 1);
      const TcItem it = tc_item(p, item);
      float mrun[8], lsum[8], acc[8];
#pragma unroll
      for (int g = 0; g < 8; ++g) { mrun[g] = -INFINITY; lsum[g] = 0.f; acc[g] = 0.f; }
      for (int t = it.t0; t < it.t1; ++t, ++m_cnt) {
        float s[8];
        good = good && __all_sync(0xffffffffu, mbar_wait(&sfull_bar[m_cnt & 1], (uint32_t)((m_cnt >> 1) & 1), abort_flag,
                                                         p.status, 740));
        if (good) {
          tc_fence_after();
          tmem_ld_32x8(tmem_base + lane_off + (uint32_t)(m_cnt & 1) * 16, s);
          tmem_ld_wait();
          const bool valid = t * 128 + row < it.len;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            s[g] = valid ? s[g] * p.scale_log2 : -INFINITY;
            const float wm = warp_max(s[g]);
            if (lane == 0) red_m[quarter * 8 + g] = wm;
          }
        }
        good = bar_and_128(good);
        if (!good) break;
        float alpha[8];
        uint8_t* prow = p_s + (row >> 6) * 2048;  // the [16 x 64 tok] tile of this token's page
        const int c = row & 63;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float tm = fmaxf(fmaxf(red_m[g], red_m[8 + g]), fmaxf(red_m[16 + g], red_m[24 + g]));
          const float mn = fmaxf(mrun[g], tm);
          alpha[g] = (mrun[g] == -INFINITY) ? 0.f : exp2f(mrun[g] - mn);
          const float pv = (s[g] == -INFINITY || g >= G) ? 0.f : exp2f(s[g] - mn);
          mrun[g] = mn;
          lsum[g] = lsum[g] * alpha[g] + pv;
          // P[g][token] as a K-major 128-byte-swizzled tile: 16-byte chunk index XOR row
          *reinterpret_cast<__nv_bfloat16*>(prow + g * 128 + ((((c >> 3) ^ g) & 7) << 4) + (c & 7) * 2) =
              __float2bfloat16(pv);
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(pfull_bar);
        good = good && __all_sync(0xffffffffu, mbar_wait(ofull_bar, (uint32_t)(m_cnt & 1), abort_flag, p.status, 750));
        if (good) {
          tc_fence_after();
          float o[8];
          tmem_ld_32x8(tmem_base + lane_off + 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 8; ++g) acc[g] = acc[g] * alpha[g] + o[g];
          tc_fence_before();
        }
      }
      if (it.t1 > it.t0) {  // every softmax thread gets here, also after a failed wait: the vote keeps them together
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float ws = warp_sum(lsum[g]);
          if (lane == 0) red_l[quarter * 8 + g] = ws;
        }
        good = bar_and_128(good);
      }
      if (!good) break;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        if (g >= G) break;
        const size_t base = ((size_t)it.b * p.Hq + it.kvh * G + g) * p.splits + it.sp;
        if (p.splits == 1) {  // nothing to merge: normalise and store the result here
          const float L = it.t1 > it.t0 ? red_l[g] + red_l[8 + g] + red_l[16 + g] + red_l[24 + g] : 0.f;
          p.out[base * 128 + row] = __float2bfloat16(L > 0.f ? acc[g] / L : 0.f);
          continue;
        }
        p.part_o[base * 128 + row] = acc[g];
        if (ts == g) {
          const bool any = it.t1 > it.t0;
          p.part_ml[base * 2] = any ? mrun[g] * LN2 : -INFINITY;
          p.part_ml[base * 2 + 1] = any ? red_l[g] + red_l[8 + g] + red_l[16 + g] + red_l[24 + g] : 0.f;
        }
      }
    }
  }

  // ---------------- teardown (also the abort path) ----------------
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TC_TMEM_COLS);
  }
}


// ---------------------------------------------------------------------------------------------------------------
// Two softmax groups.  Same tiles and data path as above, but the 128-token tiles of an item alternate between two
// groups of four warps, each with its own S^T / O^T columns in TMEM, P buffer and barriers: while group A reduces,
// exponentiates and writes P for tile n, the tensor core already runs QK^T of tile n+1 for group B and PV of tile
// n-1, so the per-tile chain (S ready -> max -> exp2 -> P -> PV -> O read) of one group hides under the other's.
// Each group keeps its own running (max, sum, O) and the two states are merged once per item through shared memory.
// ---------------------------------------------------------------------------------------------------------------
constexpr int TC2_THREADS = 320;
constexpr uint32_t TC2_TMEM_COLS = 64;                       // S0 [0,16) S1 [16,32) O0 [32,48) O1 [48,64)
constexpr uint32_t TC2_MERGE_BYTES = 128 * 8 * 4 + 64;       // group 1's O^T [8][128] fp32, max [8], sum [8]
constexpr size_t TC2_SMEM = TC_STAGES * TC_STAGE_BYTES + 2 * TC_Q_BYTES + 2 * TC_P_BYTES + 2 * TC2_MERGE_BYTES +
                            1024 /*barriers, reductions*/ + 1024 /*alignment slack*/;

__device__ __forceinline__ bool bar_and_n(bool pred, int id, int count) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "bar.red.and.pred p, %2, %3, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"((uint32_t)pred), "r"(id), "r"(count)
      : "memory");
  return out != 0;
}

__global__ void __launch_bounds__(TC2_THREADS, 1)
paged_decode_attn_tc2_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                             const TcAttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  uint8_t* q_s = smem + TC_STAGES * TC_STAGE_BYTES;  // two buffers (item parity)
  uint8_t* p_s = q_s + 2 * TC_Q_BYTES;               // one per softmax group
  uint8_t* mg_s = p_s + 2 * TC_P_BYTES;              // two buffers (item parity)
  uint64_t* bars = reinterpret_cast<uint64_t*>(mg_s + 2 * TC2_MERGE_BYTES);
  uint64_t* full_bar = bars;                    // [3]
  uint64_t* empty_bar = bars + TC_STAGES;       // [3]
  uint64_t* sfull_bar = bars + 2 * TC_STAGES;   // [2] per group
  uint64_t* pfull_bar = sfull_bar + 2;          // [2] per group
  uint64_t* ofull_bar = pfull_bar + 2;          // [2] per group
  uint64_t* qfull_bar = ofull_bar + 2;          // [2] per item parity
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(qfull_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red_m_all = reinterpret_cast<float*>(tmem_slot + 4);  // [2 groups][4][8]
  float* red_l_all = red_m_all + 64;                           // [2 groups][4][8]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_items = p.B * p.Hk * p.splits;
  const int G = p.Hq / p.Hk;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&sfull_bar[g], 1);
      mbar_init(&pfull_bar[g], 128);
      mbar_init(&ofull_bar[g], 1);
      mbar_init(&qfull_bar[g], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  // P rows 8..15 are never written by the softmax warps: zero both buffers once
  for (int i = threadIdx.x; i < (int)(2 * TC_P_BYTES / 16); i += TC2_THREADS)
    reinterpret_cast<uint4*>(p_s)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  if (warp == 1) {
    tmem_alloc(tmem_slot, TC2_TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();  // after the TMEM allocation, see common.cuh
  pdl_wait();               // q and the newest K/V rows come from the kernel before this one

  if (warp == 0) {
    // ---------------- TMA producer (same ring as the one-group kernel) ----------------
    if (lane == 0) {
      int m = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const TcItem it = tc_item(p, item);
        const int n_pages = (it.len + 63) >> 6;
        const int* bt = p.block_table + (size_t)it.slot * p.max_blocks;
        for (int t = it.t0; t < it.t1; ++t, ++m) {
          const int stage = m % TC_STAGES;
          if (!mbar_wait(&empty_bar[stage], (uint32_t)(((m / TC_STAGES) & 1) ^ 1), abort_flag, p.status, 800 + stage)) {
            ok = false;
            break;
          }
          const int pg0 = 2 * t;
          const int pg1 = (pg0 + 1 < n_pages) ? pg0 + 1 : pg0;
          const int blk0 = bt[pg0], blk1 = bt[pg1];
          uint8_t* st = stages + (size_t)stage * TC_STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], TC_STAGE_BYTES);
          for (int h = 0; h < 2; ++h) {
            tma_load_3d(st + h * 16384, &tmap_k, &full_bar[stage], h * 64, it.kvh, blk0 * 64);
            tma_load_3d(st + h * 16384 + 8192, &tmap_k, &full_bar[stage], h * 64, it.kvh, blk1 * 64);
          }
          tma_load_2d(st + 32768, &tmap_v, &full_bar[stage], 0, (blk0 * p.Hk + it.kvh) * 128);
          tma_load_2d(st + 49152, &tmap_v, &full_bar[stage], 0, (blk1 * p.Hk + it.kvh) * 128);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // Tile n of this CTA belongs to group n & 1.  Issue order: QK^T(n), QK^T(n+1), then per tile
    // [wait P(n)] PV(n), QK^T(n+2).  S^T of group g is free for QK^T(n+2) once P(n) has arrived (the group read S^T(n)
    // before writing P(n)); O^T of group g is free for PV(n) for the same reason (the group read O^T(n-2) before it
    // started on tile n).
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, 16);
      const uint32_t stages_u = smem_u32(stages), q_u = smem_u32(q_s), p_u = smem_u32(p_s);
      int m = 0, j = 0;
      bool ok = true;
      auto mma1 = [&](int mm, int jj) -> bool {
        const int stage = mm % TC_STAGES;
        if (!mbar_wait(&full_bar[stage], (uint32_t)((mm / TC_STAGES) & 1), abort_flag, p.status, 810 + stage)) return false;
        tc_fence_after();
        const uint32_t ts = tmem_base + (uint32_t)(mm & 1) * 16;
        const uint32_t kb_base = stages_u + (uint32_t)stage * TC_STAGE_BYTES, qb = q_u + (uint32_t)(jj & 1) * TC_Q_BYTES;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t adesc = umma_desc_kmajor_sw128(kb_base + kb * 16384);
          const uint64_t bdesc = umma_desc_kmajor_sw128(qb + kb * 2048);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_bf16_ss(ts, adesc + 2 * kk, bdesc + 2 * kk, idesc, (kb | kk) != 0);
        }
        umma_commit(&sfull_bar[mm & 1]);
        return true;
      };
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++j) {
        const TcItem it = tc_item(p, item);
        if (!mbar_wait(&qfull_bar[j & 1], (uint32_t)((j >> 1) & 1), abort_flag, p.status, 820)) { ok = false; break; }
        const int T = it.t1 - it.t0;
        if (T == 0) continue;
        tc_fence_after();
        if (!mma1(m, j)) { ok = false; break; }
        if (T > 1 && !mma1(m + 1, j)) { ok = false; break; }
        for (int i = 0; i < T; ++i) {
          const int mm = m + i, stage = mm % TC_STAGES, g = mm & 1;
          if (!mbar_wait(&pfull_bar[g], (uint32_t)((mm >> 1) & 1), abort_flag, p.status, 830 + g)) { ok = false; break; }
          tc_fence_after();
          const uint32_t to = tmem_base + 32 + (uint32_t)g * 16;
          const uint32_t vb = stages_u + (uint32_t)stage * TC_STAGE_BYTES + 32768;
          const uint32_t pb = p_u + (uint32_t)g * TC_P_BYTES;
#pragma unroll
          for (int pg = 0; pg < 2; ++pg) {
            const uint64_t adesc = umma_desc_kmajor_sw128(vb + pg * 16384);
            const uint64_t bdesc = umma_desc_kmajor_sw128(pb + pg * 2048);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) umma_bf16_ss(to, adesc + 2 * kk, bdesc + 2 * kk, idesc, (pg | kk) != 0);
          }
          umma_commit(&ofull_bar[g]);
          umma_commit(&empty_bar[stage]);
          if (i + 2 < T && !mma1(mm + 2, j)) { ok = false; break; }
        }
        m += T;
      }
    }
    __syncwarp();
  } else {
    // ---------------- two softmax groups of 128 threads ----------------
    const int gid = (warp - 2) >> 2;           // warps 2-5: group 0, warps 6-9: group 1
    const int quarter = warp & 3;              // TMEM lane quarter this warp may read (each group covers all four)
    const int row = quarter * 32 + lane;       // token row of S^T, head-dim row of O^T
    const int ts = (threadIdx.x - 64) & 127;   // 0..127 inside the group
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_col = tmem_base + lane_off + (uint32_t)gid * 16;
    const uint32_t o_col = tmem_base + lane_off + 32 + (uint32_t)gid * 16;
    float* red_m = red_m_all + gid * 32;
    float* red_l = red_l_all + gid * 32;
    uint8_t* p_g = p_s + (size_t)gid * TC_P_BYTES;
    constexpr float LN2 = 0.6931471805599453f;
    bool good = true;
    int n_base = 0, j = 0;

    auto write_q = [&](int item, int buf) {  // group 0 only
      const TcItem it = tc_item(p, item);
      uint8_t* dst = q_s + (size_t)buf * TC_Q_BYTES;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int ch = ts + 128 * i;          // 16 rows x 16 chunks of 8 dims
        const int r = ch >> 4, cc = ch & 15, kb = cc >> 3, c8 = cc & 7;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < G) v = *reinterpret_cast<const uint4*>(p.q + ((size_t)it.b * p.Hq + it.kvh * G + r) * 128 + cc * 8);
        *reinterpret_cast<uint4*>(dst + kb * 2048 + (r >> 3) * 1024 + (r & 7) * 128 + ((c8 ^ (r & 7)) << 4)) = v;
      }
      fence_proxy_async_smem();
      mbar_arrive(&qfull_bar[buf]);
    };

    if (gid == 0 && (int)blockIdx.x < n_items) write_q(blockIdx.x, 0);
    for (int item = blockIdx.x; item < n_items && good; item += gridDim.x, ++j) {
      // The Q buffer of the next item was last read by the item before this one; both groups passed that item's
      // merge barrier after their last O^T wait, so all of its MMAs have completed.
      if (gid == 0 && item + (int)gridDim.x < n_items) write_q(item + gridDim.x, (j + 1) & 1);
      const TcItem it = tc_item(p, item);
      const int T = it.t1 - it.t0;
      float mrun[8], lsum[8], acc[8];
#pragma unroll
      for (int g = 0; g < 8; ++g) { mrun[g] = -INFINITY; lsum[g] = 0.f; acc[g] = 0.f; }
      const int i0 = ((n_base & 1) == gid) ? 0 : 1;  // first tile of this item that belongs to this group
      const bool any = i0 < T;
      for (int i = i0; i < T; i += 2) {
        const int n = n_base + i, t = it.t0 + i;
        const uint32_t par = (uint32_t)((n >> 1) & 1);
        float s[8];
        good = good && __all_sync(0xffffffffu, mbar_wait(&sfull_bar[gid], par, abort_flag, p.status, 840 + gid));
        if (good) {
          tc_fence_after();
          tmem_ld_32x8(s_col, s);
          tmem_ld_wait();
          const bool valid = t * 128 + row < it.len;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            s[g] = valid ? s[g] * p.scale_log2 : -INFINITY;
            const float wm = warp_max(s[g]);
            if (lane == 0) red_m[quarter * 8 + g] = wm;
          }
        }
        good = bar_and_n(good, 1 + gid, 128);
        if (!good) break;
        float alpha[8];
        uint8_t* prow = p_g + (row >> 6) * 2048;  // the [16 x 64 tok] tile of this token's page
        const int c = row & 63;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float tm = fmaxf(fmaxf(red_m[g], red_m[8 + g]), fmaxf(red_m[16 + g], red_m[24 + g]));
          const float mn = fmaxf(mrun[g], tm);
          alpha[g] = (mrun[g] == -INFINITY) ? 0.f : exp2f(mrun[g] - mn);
          const float pv = (s[g] == -INFINITY || g >= G) ? 0.f : exp2f(s[g] - mn);
          mrun[g] = mn;
          lsum[g] = lsum[g] * alpha[g] + pv;
          *reinterpret_cast<__nv_bfloat16*>(prow + g * 128 + ((((c >> 3) ^ g) & 7) << 4) + (c & 7) * 2) =
              __float2bfloat16(pv);
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(&pfull_bar[gid]);
        good = good && __all_sync(0xffffffffu, mbar_wait(&ofull_bar[gid], par, abort_flag, p.status, 850 + gid));
        if (good) {
          tc_fence_after();
          float o[8];
          tmem_ld_32x8(o_col, o);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 8; ++g) acc[g] = acc[g] * alpha[g] + o[g];
          tc_fence_before();
        }
      }
      n_base += T;
      if (any) {  // uniform inside the group; reached after a failed wait too, the vote keeps the group together
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float ws = warp_sum(lsum[g]);
          if (lane == 0) red_l[quarter * 8 + g] = ws;
        }
        good = bar_and_n(good, 1 + gid, 128);
      }
      // ---- merge the two groups' states: group 1 publishes, group 0 combines and stores ----
      float* mg = reinterpret_cast<float*>(mg_s + (size_t)(j & 1) * TC2_MERGE_BYTES);
      if (gid == 1) {
        if (any && good) {
#pragma unroll
          for (int g = 0; g < 8; ++g) mg[g * 128 + row] = acc[g];
        }
        if (ts < 8) {
          mg[1024 + ts] = (any && good) ? mrun[ts] : -INFINITY;
          mg[1032 + ts] = (any && good) ? red_l[ts] + red_l[8 + ts] + red_l[16 + ts] + red_l[24 + ts] : 0.f;
        }
      }
      good = bar_and_n(good, 3, 256);  // one barrier per item: the merge buffers alternate with the item parity
      if (!good) break;
      if (gid == 1) continue;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        if (g >= G) break;
        const float m0 = any ? mrun[g] : -INFINITY, m1 = mg[1024 + g];
        const float l0 = any ? red_l[g] + red_l[8 + g] + red_l[16 + g] + red_l[24 + g] : 0.f, l1 = mg[1032 + g];
        const float M = fmaxf(m0, m1);
        const float w0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - M);
        const float w1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - M);
        float a = (m0 == -INFINITY) ? 0.f : acc[g] * w0;
        if (m1 != -INFINITY) a += mg[g * 128 + row] * w1;
        const float L = l0 * w0 + l1 * w1;
        const size_t base = ((size_t)it.b * p.Hq + it.kvh * G + g) * p.splits + it.sp;
        if (p.splits == 1) {
          p.out[base * 128 + row] = __float2bfloat16(L > 0.f ? a / L : 0.f);
          continue;
        }
        p.part_o[base * 128 + row] = a;
        if (ts == g) {
          p.part_ml[base * 2] = (T > 0) ? M * LN2 : -INFINITY;
          p.part_ml[base * 2 + 1] = (T > 0) ? L : 0.f;
        }
      }
    }
  }

  // ---------------- teardown (also the abort path) ----------------
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TC2_TMEM_COLS);
  }
}

}  // namespace trlb

using namespace trlb;

// K cache [num_blocks, 64, Hk, 128], V cache transposed per page [num_blocks, Hk, 128, 64]; G = Hq/Hk <= 8.
// scratch: part_o = B*Hq*splits*128 floats, part_ml = B*Hq*splits*2 floats.
static int decode_attn_tc_launch(const void* q, const void* kc, const void* vct, const int* seq_lens, const int* slot_ids,
                                 const int* block_table, int max_blocks, int num_blocks, int B, int Hq, int Hk, float scale,
                                 int splits, float* part_o, float* part_ml, void* out, int* status, int groups,
                                 cudaStream_t st) {
  if (B == 0) return 0;
  if (Hq % Hk != 0 || Hq / Hk > 8 || splits < 1) return -120;
  CUtensorMap tk, tv;
  int r = trlb_host::make_tmap_3d_bf16(&tk, kc, 128, (uint64_t)Hk, (uint64_t)num_blocks * 64, 128, (uint64_t)Hk * 128, 64, 1,
                                       64);
  if (r) return -121;
  r = trlb_host::make_tmap_2d_bf16(&tv, vct, (uint64_t)num_blocks * Hk * 128, 64, 64, 128, 64);
  if (r) return -122;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(paged_decode_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);
    cudaFuncSetAttribute(paged_decode_attn_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC2_SMEM);
    attr_set = true;
  }
  TcAttnParams p;
  p.q = (const __nv_bfloat16*)q; p.seq_lens = seq_lens; p.slot_ids = slot_ids; p.block_table = block_table;
  p.max_blocks = max_blocks; p.B = B; p.Hq = Hq; p.Hk = Hk; p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.part_o = part_o; p.part_ml = part_ml; p.status = status; p.out = (__nv_bfloat16*)out;
  const int items = B * Hk * splits;
  const int grid = items < trlb_host::sm_count() ? items : trlb_host::sm_count();
  const bool pdl = trlb_host::pdl_enabled();
  cudaError_t le;
  if (groups == 2)
    le = trlb_host::launch_kernel(paged_decode_attn_tc2_kernel, dim3(grid), dim3(TC2_THREADS), TC2_SMEM, st, pdl, tk, tv, p);
  else
    le = trlb_host::launch_kernel(paged_decode_attn_tc_kernel, dim3(grid), dim3(TC_THREADS), TC_SMEM, st, pdl, tk, tv, p);
  if (le != cudaSuccess) return (int)le;
  if (splits > 1)
    paged_attn_combine_kernel<128><<<B * Hq, 128, 0, st>>>(part_o, part_ml, splits, (__nv_bfloat16*)out, B * Hq);
  return (int)cudaGetLastError();
}

TRLB_API int trlb_paged_decode_attn_tc(const void* q, const void* kc, const void* vct, const int* seq_lens,
                                       const int* slot_ids, const int* block_table, int max_blocks, int num_blocks, int B,
                                       int Hq, int Hk, float scale, int splits, float* part_o, float* part_ml, void* out,
                                       int* status, cudaStream_t st) {
  return decode_attn_tc_launch(q, kc, vct, seq_lens, slot_ids, block_table, max_blocks, num_blocks, B, Hq, Hk, scale, splits,
                               part_o, part_ml, out, status, 1, st);
}

// Same operation with two softmax groups per CTA (alternating tiles); same arguments and scratch.
TRLB_API int trlb_paged_decode_attn_tc2(const void* q, const void* kc, const void* vct, const int* seq_lens,
                                        const int* slot_ids, const int* block_table, int max_blocks, int num_blocks, int B,
                                        int Hq, int Hk, float scale, int splits, float* part_o, float* part_ml, void* out,
                                        int* status, cudaStream_t st) {
  return decode_attn_tc_launch(q, kc, vct, seq_lens, slot_ids, block_table, max_blocks, num_blocks, B, Hq, Hk, scale, splits,
                               part_o, part_ml, out, status, 2, st);
}
