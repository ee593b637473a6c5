// Variable-length (packed, padding-free) causal attention for training on the 5th-generation tensor cores:
// forward, and a backward made of two kernels (dK/dV per key tile, dQ per query tile) that needs no atomics.
//
//   q [Tq, Hq, 128], k / v [Tk, Hk, 128] bf16 (row strides free: views into a fused QKV buffer work), sequences given
//   by cu_seqlens_q / cu_seqlens_k.  Grouped-query attention reads the KV head hq / (Hq / Hk) directly: K and V are
//   never expanded.  Masks: causal with the diagonal aligned to the END of the key segment (a query segment may be
//   the tail of its key segment, which is what context parallelism needs; equal lengths give the usual causal
//   mask), an optional sliding window, or none.
//
// Forward, one CTA per (128-query tile, query head), 192 threads:
//   warp 0   TMA: the Q tile once, then K tiles of 128 keys through a 3-stage ring and V tiles through a 2-stage
//            ring (a K stage is released by Q.K^T, a V stage by P.V);
//   warp 1   tcgen05.mma: S_j = Q K_j^T into one of two TMEM buffers (issued one tile ahead, so the softmax of
//            tile j runs under Q.K_{j+1}^T), then O += P_j V_j accumulating in TMEM over all key tiles.  V is
//            consumed as an MN-major operand straight from its TMA tile: no transpose anywhere;
//   warps 2-5 one thread per query row: maximum, exponentials in base 2 against a reference maximum that moves only
//            when a tile exceeds it by 2^8 (then, and only then, the warp rescales its rows of O in TMEM).  P_j goes
//            back into tensor memory as bf16 pairs over the first half of S_j's own columns and is the A operand
//            of the second MMA from there: no shared-memory tile, no proxy fence, and it is double-buffered for
//            free.  Tiles that every row sees completely skip the per-element mask tests.
//   TMEM: S0/P0 S1/P1 O = 384 columns.  Output bf16 + log-sum-exp (natural log, fp32 [Hq, Tq]) for the backward.
//
// Every wait is bounded (common.cuh); a wait that runs out reports through the status words and the CTA leaves
// through the normal teardown.
//
// Takes the place of the FlashAttention-2/3 kernels the reference reaches through transformers
// (trl/trainer/sft_trainer.py:384-390,1144-1162: padding-free batches with cu_seqlens from position_ids).
#include "common.cuh"

namespace trlb {

constexpr int FA_BM = 128, FA_BN = 128, FA_D = 128;
constexpr int FA_THREADS = 192;
constexpr uint32_t FA_TILE_BYTES = 128 * 128 * 2;  // a [128 x 128] bf16 tile = two TMA boxes of [128 rows x 64]
constexpr uint32_t FA_BOX_BYTES = 128 * 64 * 2;
// K and V tiles travel through rings of their own: a K stage is free again as soon as Q.K^T of its tile has run
// (one tile ahead of the softmax), a V stage only after P.V, so K gets the third stage and its loads start a full
// tile earlier than they could in a shared ring.
constexpr int FA_K_STAGES = 3, FA_V_STAGES = 3;
constexpr size_t FA_FWD_SMEM = FA_TILE_BYTES /*Q*/ + (FA_K_STAGES + FA_V_STAGES) * FA_TILE_BYTES + 1024 + 512;

struct FaParams {
  const int* cu_q;
  const int* cu_k;
  int n_seq, Hq, Hk;
  int causal, window;  // window <= 0: unlimited
  float scale_log2;    // softmax scale * log2(e)
  __nv_bfloat16* out;  // [Tq, Hq, 128]
  long long out_row_stride;
  float* lse;          // [Hq, Tq] natural log
  int Tq;
  int* status;
};

// Tile slot -> (sequence, query tile); tiles of a sequence are handed out from its LAST tile down, so the CTAs with
// the most keys start first.  Returns false when the slot is beyond the last tile.
__device__ __forceinline__ bool fa_find_tile(const int* cu_q, int n_seq, int slot, int& seq, int& tile) {
  for (int s = 0; s < n_seq; ++s) {
    const int nt = (cu_q[s + 1] - cu_q[s] + FA_BM - 1) / FA_BM;
    if (slot < nt) { seq = s; tile = nt - 1 - slot; return true; }
    slot -= nt;
  }
  return false;
}

// Range of key tiles [lo, hi] a query tile attends to; hi < lo means none.
__device__ __forceinline__ void fa_kv_range(int tile, int lq, int lk, int causal, int window, int& lo, int& hi) {
  const int off = lk - lq;  // key position of the diagonal for query position 0
  const int q_first = tile * FA_BM, q_last = min(lq, q_first + FA_BM) - 1;
  hi = (lk - 1) / FA_BN;
  lo = 0;
  if (causal) {
    hi = min(hi, (q_last + off) / FA_BN);
    if (q_last + off < 0) hi = -1;
    if (window > 0) lo = max(0, q_first + off - window + 1) / FA_BN;
  }
}

// byte offset of element (row r, column c) in a [128 x 128] bf16 K-major tile stored as two 128-byte-swizzled boxes
__global__ void __launch_bounds__(FA_THREADS, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
              const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  int seq, tile;
  if (!fa_find_tile(p.cu_q, p.n_seq, (int)blockIdx.x, seq, tile)) return;  // uniform: before any barrier or TMEM use
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* k_s = smem + FA_TILE_BYTES;                 // [FA_K_STAGES] K tiles
  uint8_t* v_s = k_s + FA_K_STAGES * FA_TILE_BYTES;    // [FA_V_STAGES] V tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + FA_V_STAGES * FA_TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                  // [FA_K_STAGES]
  uint64_t* k_empty = k_full + FA_K_STAGES;     // [FA_K_STAGES]
  uint64_t* v_full = k_empty + FA_K_STAGES;     // [FA_V_STAGES]
  uint64_t* v_empty = v_full + FA_V_STAGES;     // [FA_V_STAGES]
  uint64_t* s_full = v_empty + FA_V_STAGES;     // [2]
  uint64_t* o_full = s_full + 2;                // one phase per P.V product
  uint64_t* p_full = o_full + 1;                // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_full + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, kvh = h / (p.Hq / p.Hk);
  const int q_beg = p.cu_q[seq], lq = p.cu_q[seq + 1] - q_beg;
  const int k_beg = p.cu_k[seq], lk = p.cu_k[seq + 1] - k_beg;
  int lo, hi;
  fa_kv_range(tile, lq, lk, p.causal, p.window, lo, hi);
  const int n_kv = hi - lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < FA_K_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < FA_V_STAGES; ++s) {
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 128);
    }
    mbar_init(o_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (n_kv > 0) {
    if (warp == 0) {
      // ---------------- TMA producer ----------------
      if (lane == 0) {
        mbar_expect_tx(q_full, FA_TILE_BYTES);
        tma_load_2d(q_s, &tmap_q, q_full, h * FA_D, q_beg + tile * FA_BM);
        tma_load_2d(q_s + FA_BOX_BYTES, &tmap_q, q_full, h * FA_D + 64, q_beg + tile * FA_BM);
        auto load_k = [&](int j) {
          const int s = j % FA_K_STAGES;
          if (!mbar_wait(&k_empty[s], (uint32_t)(((j / FA_K_STAGES) & 1) ^ 1), abort_flag, p.status, 1000 + s)) return false;
          uint8_t* ks = k_s + (size_t)s * FA_TILE_BYTES;
          const int row = k_beg + (lo + j) * FA_BN;
          mbar_expect_tx(&k_full[s], FA_TILE_BYTES);
          tma_load_2d(ks, &tmap_k, &k_full[s], kvh * FA_D, row);
          tma_load_2d(ks + FA_BOX_BYTES, &tmap_k, &k_full[s], kvh * FA_D + 64, row);
          return true;
        };
        // order K(0) K(1) V(0) K(2) V(1) ...: a V stage frees later than the K stage asked for after it
        bool ok = load_k(0);
        for (int j = 0; j < n_kv && ok; ++j) {
          if (j + 1 < n_kv) ok = load_k(j + 1);
          if (!ok) break;
          const int s = j % FA_V_STAGES;
          if (!mbar_wait(&v_empty[s], (uint32_t)(((j / FA_V_STAGES) & 1) ^ 1), abort_flag, p.status, 1005 + s)) break;
          uint8_t* vs = v_s + (size_t)s * FA_TILE_BYTES;
          const int row = k_beg + (lo + j) * FA_BN;
          mbar_expect_tx(&v_full[s], FA_TILE_BYTES);
          tma_load_2d(vs, &tmap_v, &v_full[s], kvh * FA_D, row);
          tma_load_2d(vs + FA_BOX_BYTES, &tmap_v, &v_full[s], kvh * FA_D + 64, row);
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // ---------------- MMA issuer ----------------
      if (lane == 0) {
        constexpr uint32_t idesc_s = umma_idesc_bf16_major(FA_BM, FA_BN, false, false);
        constexpr uint32_t idesc_o = umma_idesc_bf16_major(FA_BM, FA_D, false, true);  // V is MN-major
        const uint32_t q_u = smem_u32(q_s), ks_u = smem_u32(k_s), vs_u = smem_u32(v_s);
        bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 1010);
        auto issue_s = [&](int j) {
          const int s = j & 1, kst = j % FA_K_STAGES;  // TMEM buffer, K ring stage
          // buffer s is free: it held S and then P of tile j - 2, whose P.V product was issued before this call
          if (!mbar_wait(&k_full[kst], (uint32_t)((j / FA_K_STAGES) & 1), abort_flag, p.status, 1020 + kst)) return false;
          tc_fence_after();
          const uint32_t k_u = ks_u + (uint32_t)kst * FA_TILE_BYTES;
#pragma unroll
          for (int kk = 0; kk < FA_D / 16; ++kk) {
            const uint32_t off = (uint32_t)(kk >> 2) * FA_BOX_BYTES;
            umma_bf16_ss(tmem_base + (uint32_t)s * FA_BN, umma_desc_kmajor_sw128(q_u + off) + 2 * (kk & 3),
                         umma_desc_kmajor_sw128(k_u + off) + 2 * (kk & 3), idesc_s, kk != 0);
          }
          umma_commit(&s_full[s]);
          umma_commit(&k_empty[kst]);
          return true;
        };
        if (ok) ok = issue_s(0);
        for (int j = 0; j < n_kv && ok; ++j) {
          const int s = j % FA_V_STAGES;
          if (j + 1 < n_kv) ok = issue_s(j + 1);
          if (!ok) break;
          const int sb = j & 1;  // the TMEM buffer that held S_j now holds P_j (bf16 pairs in its first 64 columns)
          if (!mbar_wait(&p_full[sb], (uint32_t)((j >> 1) & 1), abort_flag, p.status, 1040 + sb)) { ok = false; break; }
          if (!mbar_wait(&v_full[s], (uint32_t)((j / FA_V_STAGES) & 1), abort_flag, p.status, 1050 + s)) { ok = false; break; }
          tc_fence_after();
          const uint32_t v_u = vs_u + (uint32_t)s * FA_TILE_BYTES;
#pragma unroll
          for (int kk = 0; kk < FA_BN / 16; ++kk) {
            const uint64_t bdesc = umma_desc_mnmajor_sw128(v_u + (uint32_t)kk * 2048, FA_BOX_BYTES);
            // P is the A operand straight from tensor memory (16 keys = 8 columns per step).  O accumulates in TMEM
            // over all key tiles; the row threads rescale it in place when a row's reference maximum moves (see
            // below), always between two P.V products
            umma_bf16_ts(tmem_base + 256, tmem_base + (uint32_t)sb * FA_BN + (uint32_t)kk * 8, bdesc, idesc_o,
                         (j != 0) || (kk != 0));
          }
          umma_commit(o_full);
          umma_commit(&v_empty[s]);
        }
      }
      __syncwarp();
    } else {
      // ---------------- softmax: one thread per query row ----------------
      // The output accumulates in TMEM.  A row keeps a *reference* maximum m_ref for its exponents and moves it only
      // when a tile's maximum exceeds it by more than 8 (in log2 units): until then probabilities are at most 2^8,
      // which bf16 and the fp32 sums hold without loss, and nothing has to be rescaled.  When it does move, the
      // warp rescales its 32 rows of O in TMEM (after the previous P.V product has finished, before the next one is
      // released) and the running sum; with ordinary scores that happens in the first tile or two of a row only.
      const int quarter = warp & 3;
      const int r = quarter * 32 + lane;
      const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
      const int q_first = tile * FA_BM;
      const int q_pos = q_first + r;  // position inside the query segment
      const bool row_ok = q_pos < lq;
      const int off = lk - lq;
      // keys this row may see: [k_min, k_max]
      const int k_max = p.causal ? min(lk - 1, q_pos + off) : lk - 1;
      const int k_min = (p.causal && p.window > 0) ? max(0, q_pos + off - p.window + 1) : 0;
      const uint32_t to = tmem_base + lane_off + 256;
      float m_ref = -INFINITY, l_run = 0.f;
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        const int key0 = (lo + j) * FA_BN;
        // every row of the tile sees every key of this tile: no per-element tests (all but the diagonal / edge tiles)
        bool full = (q_first + FA_BM <= lq) && (key0 + FA_BN <= lk);
        if (p.causal) {
          full = full && (key0 + FA_BN - 1 <= q_first + off);
          if (p.window > 0) full = full && (key0 >= q_first + FA_BM - 1 + off - p.window + 1);
        }
        ok = __all_sync(0xffffffffu, mbar_wait(&s_full[s], (uint32_t)((j >> 1) & 1), abort_flag, p.status, 1070 + s));
        if (!ok) break;
        tc_fence_after();
        const uint32_t ts = tmem_base + lane_off + (uint32_t)s * FA_BN;
        // pass 1: row maximum over this tile's visible keys (raw scores; the scale is positive)
        float mx = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < FA_BN; c += 64) {
          float v0[32], v1[32];
          tmem_ld_32x32(ts + c, v0);
          tmem_ld_32x32(ts + c + 32, v1);
          tmem_ld_wait();
          if (full) {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(v0[i], v1[i]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int key = key0 + c + i;
              if (row_ok && key >= k_min && key <= k_max) mx = fmaxf(mx, v0[i]);
              if (row_ok && key + 32 >= k_min && key + 32 <= k_max) mx = fmaxf(mx, v1[i]);
            }
          }
        }
        const float m_tile = mx * p.scale_log2;
        float alpha = 1.f;
        bool moved = false;
        if (m_ref == -INFINITY) {
          m_ref = m_tile;  // nothing seen so far: the row of O is still zero, nothing to rescale
        } else if (m_tile > m_ref + 8.f) {
          alpha = fast_exp2(m_ref - m_tile);
          m_ref = m_tile;
          moved = true;
        }
        if (j > 0 && __any_sync(0xffffffffu, moved)) {
          // P.V of tile j-1 must have landed; the tile before it has (S of this tile was issued after it)
          ok = __all_sync(0xffffffffu, mbar_wait(o_full, (uint32_t)((j - 1) & 1), abort_flag, p.status, 1090));
          if (!ok) break;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < FA_D; c += 32) {
            float v[32];
            tmem_ld_32x32(to + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= alpha;
            tmem_st_32x32(to + c, v);
          }
          tmem_st_wait();
        }
        l_run *= alpha;
        const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
        // pass 2: probabilities, row sum; P_j (bf16 pairs) overwrites the columns of S_j this thread has already read
        float sum = 0.f;
#pragma unroll 1
        for (int c = 0; c < FA_BN; c += 32) {
          float v[32];
          tmem_ld_32x32(ts + c, v);
          tmem_ld_wait();
          if (full) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              v[i] = fast_exp2(fmaf(v[i], p.scale_log2, neg_m));
              sum += v[i];
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int key = key0 + c + i;
              const bool vis = row_ok && key >= k_min && key <= k_max;
              v[i] = vis ? fast_exp2(fmaf(v[i], p.scale_log2, neg_m)) : 0.f;
              sum += v[i];
            }
          }
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) w[i] = pack_bf16(v[2 * i], v[2 * i + 1]);
          tmem_st_32x16(ts + (c >> 1), w);
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&p_full[s]);
        l_run += sum;
      }
      if (ok) {
        // the last P.V product: wait for the one before it first, so that the parity of the last wait is unambiguous
        const int last = n_kv - 1;
        if (last >= 1)
          ok = __all_sync(0xffffffffu, mbar_wait(o_full, (uint32_t)((last - 1) & 1), abort_flag, p.status, 1094));
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(o_full, (uint32_t)(last & 1), abort_flag, p.status, 1095));
        if (ok) {
          tc_fence_after();
          const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
          __nv_bfloat16* dst = p.out + (long long)(q_beg + q_pos) * p.out_row_stride + (long long)h * FA_D;
#pragma unroll 1
          for (int c = 0; c < FA_D; c += 32) {
            float v[32];
            tmem_ld_32x32(to + c, v);
            tmem_ld_wait();
            if (row_ok) {
#pragma unroll
              for (int i = 0; i < 32; i += 8)
                *reinterpret_cast<uint4*>(dst + c + i) =
                    make_uint4(pack_bf16(v[i] * inv, v[i + 1] * inv), pack_bf16(v[i + 2] * inv, v[i + 3] * inv),
                               pack_bf16(v[i + 4] * inv, v[i + 5] * inv), pack_bf16(v[i + 6] * inv, v[i + 7] * inv));
            }
          }
          tc_fence_before();
          if (row_ok && p.lse != nullptr)
            p.lse[(long long)h * p.Tq + q_beg + q_pos] =
                l_run > 0.f ? (m_ref + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
        }
      }
    }
  } else if (warp >= 2) {
    // no visible key at all (a query segment longer than its key segment): zeros, log-sum-exp -inf
    const int r = (warp & 3) * 32 + lane;
    const int q_pos = tile * FA_BM + r;
    if (q_pos < lq) {
      __nv_bfloat16* dst = p.out + (long long)(q_beg + q_pos) * p.out_row_stride + (long long)h * FA_D;
      for (int i = 0; i < FA_D; i += 8) *reinterpret_cast<uint4*>(dst + i) = make_uint4(0, 0, 0, 0);
      if (p.lse != nullptr) p.lse[(long long)h * p.Tq + q_beg + q_pos] = -INFINITY;
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

// q [Tq, Hq, 128] / k, v [Tk, Hk, 128] bf16 with row strides q_rs / k_rs / v_rs (elements; the head dimension is
// contiguous and heads are 128 elements apart), cu_q / cu_k [n_seq + 1] int32 on the device.  out [Tq, Hq, 128] bf16
// (row stride o_rs), lse [Hq, Tq] fp32 or null.  causal: the diagonal is aligned to the end of each key segment;
// window > 0 limits every query to its last `window` keys.
TRLB_API int trlb_fa_varlen_fwd(const void* q, const void* k, const void* v, long long q_rs, long long k_rs, long long v_rs,
                                const int* cu_q, const int* cu_k, int n_seq, int Tq, int Tk, int Hq, int Hk, int D,
                                float scale, int causal, int window, void* out, long long o_rs, float* lse, int* status,
                                cudaStream_t st) {
  if (Tq <= 0 || n_seq <= 0) return 0;
  if (D != FA_D || Hk <= 0 || Hq % Hk != 0 || (q_rs % 8) || (k_rs % 8) || (v_rs % 8) || (o_rs % 8)) return -160;
  CUtensorMap tq, tk, tv;
  if (trlb_host::make_tmap_2d_bf16(&tq, q, (uint64_t)Tq, (uint64_t)Hq * D, (uint64_t)q_rs, FA_BM, 64)) return -161;
  if (trlb_host::make_tmap_2d_bf16(&tk, k, (uint64_t)Tk, (uint64_t)Hk * D, (uint64_t)k_rs, FA_BN, 64)) return -162;
  if (trlb_host::make_tmap_2d_bf16(&tv, v, (uint64_t)Tk, (uint64_t)Hk * D, (uint64_t)v_rs, FA_BN, 64)) return -163;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(fa_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FA_FWD_SMEM) != cudaSuccess)
      return -164;
    attr_set = true;
  }
  FaParams p = {};
  p.cu_q = cu_q; p.cu_k = cu_k; p.n_seq = n_seq; p.Hq = Hq; p.Hk = Hk; p.causal = causal; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.out = (__nv_bfloat16*)out; p.out_row_stride = o_rs; p.lse = lse; p.Tq = Tq; p.status = status;
  const int max_tiles = (Tq + FA_BM - 1) / FA_BM + n_seq;  // every sequence adds at most one partial tile
  fa_fwd_kernel<<<dim3(max_tiles, Hq), FA_THREADS, FA_FWD_SMEM, st>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}

// =====================================================================================================================
// Backward.  With P = softmax(S), S = scale * Q K^T, delta_i = sum_d dO_id O_id:
//     dV = P^T dO        dP = dO V^T        dS = P o (dP - delta) * scale        dQ = dS K        dK = dS^T Q
// Two kernels share no accumulator, so nothing is added atomically:
//   fa_bwd_dq_kernel   one CTA per (128-query tile, query head); walks the visible keys in chunks of 64:
//                      S = Q K_c^T and dP = dO V_c^T into TMEM (double-buffered), the row threads form dS (bf16
//                      pairs written back over S in TMEM), dQ += dS K_c accumulates in TMEM (dS as the A operand
//                      from tensor memory, K_c as an MN-major operand).
//   fa_bwd_dkv_kernel  one CTA per (128-key tile, KV head); walks the query heads of the group and, for each, the
//                      queries that see the tile in chunks of 64: S^T = K Q_c^T and dP^T = V dO_c^T into TMEM, the
//                      row threads (one per key) form P^T and dS^T, dV += P^T dO_c and dK += dS^T Q_c accumulate in
//                      TMEM over all chunks and all heads of the group (this is where grouped-query gradients are
//                      summed), dO_c / Q_c as MN-major operands.
// Probabilities are recomputed from the saved log-sum-exp: P = exp2(S * scale * log2e - lse * log2e).
// =====================================================================================================================
namespace trlb {

constexpr int FB_C = 64;                                  // inner chunk (keys for dQ, queries for dK/dV)
constexpr uint32_t FB_CHUNK_BYTES = FB_C * 128 * 2;       // [64 x 128] bf16 = two boxes of [64 rows x 64]
constexpr uint32_t FB_CBOX_BYTES = FB_C * 64 * 2;
// The chunk rings are deeper than the two TMEM buffers they feed: a stage is refilled only when the second MMA of
// its chunk has finished, and a TMA round trip (L2 or HBM to shared memory) is longer than the work on one chunk.
// dS (and P^T, dS^T in the other kernel) never visit shared memory: the row threads write them as bf16 pairs over the
// tensor-memory columns of S / dP they have just read, and the second MMA takes them as its A operand from there.
constexpr int FB_QD_STAGES = 4;  // dK/dV kernel: ring of (Q chunk, dO chunk) pairs
constexpr int FB_KV_STAGES = 5;  // dQ kernel: ring of (K chunk, V chunk) pairs
constexpr size_t FA_DQ_SMEM = 2 * FA_TILE_BYTES + FB_KV_STAGES * 2 * FB_CHUNK_BYTES + 1024 + 512;
constexpr size_t FA_DKV_SMEM = 2 * FA_TILE_BYTES + FB_QD_STAGES * 2 * FB_CHUNK_BYTES + FB_QD_STAGES * 2 * FB_C * 4 + 1024 + 512;

struct FaBwdParams {
  const int* cu_q;
  const int* cu_k;
  int n_seq, Hq, Hk, causal, window;
  float scale, scale_log2;
  const float* lse;    // [Hq, Tq] natural log
  const float* delta;  // [Hq, Tq]
  int Tq, Tk;
  __nv_bfloat16* dq;   // [Tq, Hq, 128]
  __nv_bfloat16* dk;   // [Tk, Hk, 128]
  __nv_bfloat16* dv;
  long long dq_rs, dk_rs, dv_rs;
  int* status;
};

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (t, h)
__global__ void __launch_bounds__(256)
fa_delta_kernel(const __nv_bfloat16* __restrict__ dout, long long do_rs, const __nv_bfloat16* __restrict__ out,
                long long o_rs, float* __restrict__ delta, int Tq, int Hq) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < (long long)Tq * Hq; w += warps) {
    const int t = (int)(w / Hq), h = (int)(w % Hq);
    const uint2 a = *reinterpret_cast<const uint2*>(dout + (long long)t * do_rs + h * FA_D + lane * 4);
    const uint2 b = *reinterpret_cast<const uint2*>(out + (long long)t * o_rs + h * FA_D + lane * 4);
    const float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), b0 = unpack_bf16(b.x), b1 = unpack_bf16(b.y);
    const float s = warp_sum(a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y);
    if (lane == 0) delta[(long long)h * Tq + t] = s;
  }
}

__global__ void __launch_bounds__(FA_THREADS, 1)
fa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                 const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                 const FaBwdParams p) {
  int seq, tile;
  if (!fa_find_tile(p.cu_q, p.n_seq, (int)blockIdx.x, seq, tile)) return;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* do_s = smem + FA_TILE_BYTES;
  uint8_t* kv_s = smem + 2 * FA_TILE_BYTES;  // stage s: K chunk then V chunk
  uint64_t* bars = reinterpret_cast<uint64_t*>(kv_s + FB_KV_STAGES * 2 * FB_CHUNK_BYTES);
  uint64_t* qdo_full = bars;
  uint64_t* kv_full = bars + 1;                      // [FB_KV_STAGES]
  uint64_t* kv_empty = kv_full + FB_KV_STAGES;       // [FB_KV_STAGES]
  uint64_t* sp_full = kv_empty + FB_KV_STAGES;       // [2]  S and dP of a chunk are complete
  uint64_t* ds_full = sp_full + 2;                   // [2]  dS of a chunk is in tensor memory
  uint64_t* dq_done = ds_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dq_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, kvh = h / (p.Hq / p.Hk);
  const int q_beg = p.cu_q[seq], lq = p.cu_q[seq + 1] - q_beg;
  const int k_beg = p.cu_k[seq], lk = p.cu_k[seq + 1] - k_beg;
  int lo, hi;
  fa_kv_range(tile, lq, lk, p.causal, p.window, lo, hi);
  // the forward's range is in 128-key tiles; here chunks of 64
  const int c_lo = lo * 2, c_hi = min(hi * 2 + 1, (lk - 1) / FB_C);
  const int n_c = hi < lo ? 0 : c_hi - c_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int s = 0; s < FB_KV_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sp_full[s], 1);
      mbar_init(&ds_full[s], 128);
    }
    mbar_init(dq_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_do);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: S0 [0,64) dP0 [64,128) S1 [128,192) dP1 [192,256) dQ [256,384)

  if (n_c > 0) {
    if (warp == 0) {
      if (lane == 0) {
        const int qrow = q_beg + tile * FA_BM;
        mbar_expect_tx(qdo_full, 2 * FA_TILE_BYTES);
        tma_load_2d(q_s, &tmap_q, qdo_full, h * FA_D, qrow);
        tma_load_2d(q_s + FA_BOX_BYTES, &tmap_q, qdo_full, h * FA_D + 64, qrow);
        tma_load_2d(do_s, &tmap_do, qdo_full, h * FA_D, qrow);
        tma_load_2d(do_s + FA_BOX_BYTES, &tmap_do, qdo_full, h * FA_D + 64, qrow);
        for (int j = 0; j < n_c; ++j) {
          const int s = j % FB_KV_STAGES;
          if (!mbar_wait(&kv_empty[s], (uint32_t)(((j / FB_KV_STAGES) & 1) ^ 1), abort_flag, p.status, 1100 + s)) break;
          uint8_t* ks = kv_s + (size_t)s * 2 * FB_CHUNK_BYTES;
          uint8_t* vs = ks + FB_CHUNK_BYTES;
          const int row = k_beg + (c_lo + j) * FB_C;
          mbar_expect_tx(&kv_full[s], 2 * FB_CHUNK_BYTES);
          tma_load_2d(ks, &tmap_k, &kv_full[s], kvh * FA_D, row);
          tma_load_2d(ks + FB_CBOX_BYTES, &tmap_k, &kv_full[s], kvh * FA_D + 64, row);
          tma_load_2d(vs, &tmap_v, &kv_full[s], kvh * FA_D, row);
          tma_load_2d(vs + FB_CBOX_BYTES, &tmap_v, &kv_full[s], kvh * FA_D + 64, row);
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      if (lane == 0) {
        constexpr uint32_t idesc_s = umma_idesc_bf16_major(FA_BM, FB_C, false, false);
        constexpr uint32_t idesc_dq = umma_idesc_bf16_major(FA_BM, FA_D, false, true);  // K chunk as MN-major operand
        const uint32_t q_u = smem_u32(q_s), do_u = smem_u32(do_s), kv_u = smem_u32(kv_s);
        bool ok = mbar_wait(qdo_full, 0, abort_flag, p.status, 1110);
        auto issue_sp = [&](int j) {
          const int s = j & 1, ks = j % FB_KV_STAGES;  // TMEM buffer, ring stage
          // TMEM buffer s is free: the dQ product of chunk j - 2, which read dS from it, was issued before this call
          if (!mbar_wait(&kv_full[ks], (uint32_t)((j / FB_KV_STAGES) & 1), abort_flag, p.status, 1120 + ks)) return false;
          tc_fence_after();
          const uint32_t k_u = kv_u + (uint32_t)ks * 2 * FB_CHUNK_BYTES, v_u = k_u + FB_CHUNK_BYTES;
#pragma unroll
          for (int kk = 0; kk < FA_D / 16; ++kk) {
            const uint32_t qo = (uint32_t)(kk >> 2) * FA_BOX_BYTES, co = (uint32_t)(kk >> 2) * FB_CBOX_BYTES;
            umma_bf16_ss(tmem_base + (uint32_t)s * 128, umma_desc_kmajor_sw128(q_u + qo) + 2 * (kk & 3),
                         umma_desc_kmajor_sw128(k_u + co) + 2 * (kk & 3), idesc_s, kk != 0);
          }
#pragma unroll
          for (int kk = 0; kk < FA_D / 16; ++kk) {
            const uint32_t qo = (uint32_t)(kk >> 2) * FA_BOX_BYTES, co = (uint32_t)(kk >> 2) * FB_CBOX_BYTES;
            umma_bf16_ss(tmem_base + (uint32_t)s * 128 + 64, umma_desc_kmajor_sw128(do_u + qo) + 2 * (kk & 3),
                         umma_desc_kmajor_sw128(v_u + co) + 2 * (kk & 3), idesc_s, kk != 0);
          }
          umma_commit(&sp_full[s]);
          return true;
        };
        if (ok) ok = issue_sp(0);
        for (int j = 0; j < n_c && ok; ++j) {
          const int s = j % FB_KV_STAGES;
          if (j + 1 < n_c) ok = issue_sp(j + 1);
          if (!ok) break;
          const int sb = j & 1;
          if (!mbar_wait(&ds_full[sb], (uint32_t)((j >> 1) & 1), abort_flag, p.status, 1140 + sb)) { ok = false; break; }
          tc_fence_after();
          const uint32_t k_u = kv_u + (uint32_t)s * 2 * FB_CHUNK_BYTES;
#pragma unroll
          for (int kk = 0; kk < FB_C / 16; ++kk)
            umma_bf16_ts(tmem_base + 256, tmem_base + (uint32_t)sb * 128 + (uint32_t)kk * 8,
                         umma_desc_mnmajor_sw128(k_u + (uint32_t)kk * 2048, FB_CBOX_BYTES), idesc_dq, (j | kk) != 0);
          umma_commit(&kv_empty[s]);
        }
        if (ok) umma_commit(dq_done);
      }
      __syncwarp();
    } else {
      const int quarter = warp & 3;
      const int r = quarter * 32 + lane;
      const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
      const int q_pos = tile * FA_BM + r;
      const bool row_ok = q_pos < lq;
      const int off = lk - lq;
      const int k_max = p.causal ? min(lk - 1, q_pos + off) : lk - 1;
      const int k_min = (p.causal && p.window > 0) ? max(0, q_pos + off - p.window + 1) : 0;
      float lse2 = INFINITY, dl = 0.f;
      if (row_ok) {
        const float l = p.lse[(long long)h * p.Tq + q_beg + q_pos];
        lse2 = l == -INFINITY ? INFINITY : l * 1.4426950408889634f;
        dl = p.delta[(long long)h * p.Tq + q_beg + q_pos];
      }
      const float neg_lse = -lse2;
      const int q_first = tile * FA_BM;
      bool ok = true;
      for (int j = 0; j < n_c && ok; ++j) {
        const int s = j & 1;
        const int key0 = (c_lo + j) * FB_C;
        bool full = (q_first + FA_BM <= lq) && (key0 + FB_C <= lk);
        if (p.causal) {
          full = full && (key0 + FB_C - 1 <= q_first + off);
          if (p.window > 0) full = full && (key0 >= q_first + FA_BM - 1 + off - p.window + 1);
        }
        ok = __all_sync(0xffffffffu, mbar_wait(&sp_full[s], (uint32_t)((j >> 1) & 1), abort_flag, p.status, 1150 + s));
        if (!ok) break;
        tc_fence_after();
        const uint32_t ts = tmem_base + lane_off + (uint32_t)s * 128;
#pragma unroll 1
        for (int c = 0; c < FB_C; c += 32) {
          float sv[32], dp[32];
          tmem_ld_32x32(ts + c, sv);
          tmem_ld_32x32(ts + 64 + c, dp);
          tmem_ld_wait();
          if (full) {  // every row sees every key of the chunk
#pragma unroll
            for (int i = 0; i < 32; ++i)
              sv[i] = fast_exp2(fmaf(sv[i], p.scale_log2, neg_lse)) * ((dp[i] - dl) * p.scale);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int key = key0 + c + i;
              const bool a = row_ok && key >= k_min && key <= k_max;
              sv[i] = a ? fast_exp2(fmaf(sv[i], p.scale_log2, neg_lse)) * ((dp[i] - dl) * p.scale) : 0.f;
            }
          }
          uint32_t w[16];  // dS as bf16 pairs over the columns of S already read
#pragma unroll
          for (int i = 0; i < 16; ++i) w[i] = pack_bf16(sv[2 * i], sv[2 * i + 1]);
          tmem_st_32x16(ts + (c >> 1), w);
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&ds_full[s]);
      }
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(dq_done, 0, abort_flag, p.status, 1170));
      if (ok) {
        tc_fence_after();
        __nv_bfloat16* dst = p.dq + (long long)(q_beg + q_pos) * p.dq_rs + (long long)h * FA_D;
#pragma unroll 1
        for (int c = 0; c < FA_D; c += 32) {
          float v[32];
          tmem_ld_32x32(tmem_base + lane_off + 256 + c, v);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8)
              *reinterpret_cast<uint4*>(dst + c + i) = make_uint4(pack_bf16(v[i], v[i + 1]), pack_bf16(v[i + 2], v[i + 3]),
                                                                  pack_bf16(v[i + 4], v[i + 5]), pack_bf16(v[i + 6], v[i + 7]));
          }
        }
        tc_fence_before();
      }
    }
  } else if (warp >= 2) {
    const int r = (warp & 3) * 32 + lane;
    const int q_pos = tile * FA_BM + r;
    if (q_pos < lq) {
      __nv_bfloat16* dst = p.dq + (long long)(q_beg + q_pos) * p.dq_rs + (long long)h * FA_D;
      for (int i = 0; i < FA_D; i += 8) *reinterpret_cast<uint4*>(dst + i) = make_uint4(0, 0, 0, 0);
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

// Tile slot -> (sequence, key tile); same order as fa_find_tile, on the key segments.
__device__ __forceinline__ bool fa_find_ktile(const int* cu_k, int n_seq, int slot, int& seq, int& tile) {
  for (int s = 0; s < n_seq; ++s) {
    const int nt = (cu_k[s + 1] - cu_k[s] + FA_BN - 1) / FA_BN;
    if (slot < nt) { seq = s; tile = slot; return true; }
    slot -= nt;
  }
  return false;
}

__global__ void __launch_bounds__(FA_THREADS, 1)
fa_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                  const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                  const FaBwdParams p) {
  int seq, tile;
  if (!fa_find_ktile(p.cu_k, p.n_seq, (int)blockIdx.x, seq, tile)) return;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_s = smem;
  uint8_t* v_s = smem + FA_TILE_BYTES;
  uint8_t* qd_s = smem + 2 * FA_TILE_BYTES;      // stage s: Q chunk then dO chunk
  float* stat_s = reinterpret_cast<float*>(qd_s + FB_QD_STAGES * 2 * FB_CHUNK_BYTES);  // [stage][lse2 x 64, delta x 64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(stat_s + FB_QD_STAGES * 2 * FB_C);
  uint64_t* kv_full = bars;
  uint64_t* qd_full = bars + 1;                  // [FB_QD_STAGES]
  uint64_t* qd_empty = qd_full + FB_QD_STAGES;   // [FB_QD_STAGES]
  uint64_t* sp_full = qd_empty + FB_QD_STAGES;   // [2]
  uint64_t* pd_full = sp_full + 2;               // [2]  P^T and dS^T of a chunk are in tensor memory
  uint64_t* acc_done = pd_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.y, G = p.Hq / p.Hk;
  const int q_beg = p.cu_q[seq], lq = p.cu_q[seq + 1] - q_beg;
  const int k_beg = p.cu_k[seq], lk = p.cu_k[seq + 1] - k_beg;
  const int off = lk - lq;
  const int key_first = tile * FA_BN, key_last = min(lk, key_first + FA_BN) - 1;
  // queries that see at least one key of this tile: q + off >= key_first, and with a window q + off - window < key_last
  int qc_lo = 0, qc_hi = (lq - 1) / FB_C;
  if (p.causal) {
    qc_lo = max(0, key_first - off) / FB_C;
    if (p.window > 0) qc_hi = min(qc_hi, max(0, key_last + p.window - 1 - off) / FB_C);
  }
  const int per_head = (lq > 0 && qc_hi >= qc_lo) ? qc_hi - qc_lo + 1 : 0;
  const int n_it = per_head * G;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < FB_QD_STAGES; ++s) {
      mbar_init(&qd_full[s], 33);  // the TMA transaction + 32 lanes that stage lse / delta
      mbar_init(&qd_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sp_full[s], 1);
      mbar_init(&pd_full[s], 128);
    }
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_do);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: S^T0 [0,64) dP^T0 [64,128) S^T1 [128,192) dP^T1 [192,256) dV [256,384) dK [384,512)

  if (n_it > 0) {
    if (warp == 0) {
      if (lane == 0) {
        const int krow = k_beg + tile * FA_BN;
        mbar_expect_tx(kv_full, 2 * FA_TILE_BYTES);
        tma_load_2d(k_s, &tmap_k, kv_full, kvh * FA_D, krow);
        tma_load_2d(k_s + FA_BOX_BYTES, &tmap_k, kv_full, kvh * FA_D + 64, krow);
        tma_load_2d(v_s, &tmap_v, kv_full, kvh * FA_D, krow);
        tma_load_2d(v_s + FA_BOX_BYTES, &tmap_v, kv_full, kvh * FA_D + 64, krow);
      }
      bool ok = true;
      for (int j = 0; j < n_it && ok; ++j) {
        const int s = j % FB_QD_STAGES;
        const int h = kvh * G + j / per_head, qc = qc_lo + j % per_head;
        ok = __all_sync(0xffffffffu, mbar_wait(&qd_empty[s], (uint32_t)(((j / FB_QD_STAGES) & 1) ^ 1), abort_flag, p.status, 1200 + s));
        if (!ok) break;
        if (lane == 0) {  // the bulk copies first: the scalar loads below then run under their latency
          uint8_t* qs = qd_s + (size_t)s * 2 * FB_CHUNK_BYTES;
          uint8_t* ds = qs + FB_CHUNK_BYTES;
          const int row = q_beg + qc * FB_C;
          mbar_expect_tx(&qd_full[s], 2 * FB_CHUNK_BYTES);
          tma_load_2d(qs, &tmap_q, &qd_full[s], h * FA_D, row);
          tma_load_2d(qs + FB_CBOX_BYTES, &tmap_q, &qd_full[s], h * FA_D + 64, row);
          tma_load_2d(ds, &tmap_do, &qd_full[s], h * FA_D, row);
          tma_load_2d(ds + FB_CBOX_BYTES, &tmap_do, &qd_full[s], h * FA_D + 64, row);
        }
        __syncwarp();
        float* st = stat_s + s * 2 * FB_C;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int qp = qc * FB_C + lane + 32 * u;
          float l2 = INFINITY, dl = 0.f;  // a query beyond the segment gets probability 0 everywhere
          if (qp < lq) {
            const float l = p.lse[(long long)h * p.Tq + q_beg + qp];
            l2 = l == -INFINITY ? INFINITY : l * 1.4426950408889634f;
            dl = p.delta[(long long)h * p.Tq + q_beg + qp];
          }
          st[lane + 32 * u] = l2;
          st[FB_C + lane + 32 * u] = dl;
        }
        mbar_arrive(&qd_full[s]);  // this lane's lse / delta are in shared memory (release)
      }
    } else if (warp == 1) {
      if (lane == 0) {
        constexpr uint32_t idesc_st = umma_idesc_bf16_major(FA_BN, FB_C, false, false);
        constexpr uint32_t idesc_acc = umma_idesc_bf16_major(FA_BN, FA_D, false, true);  // dO / Q chunks MN-major
        const uint32_t k_u = smem_u32(k_s), v_u = smem_u32(v_s), qd_u = smem_u32(qd_s);
        bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, 1210);
        auto issue_sp = [&](int j) {
          const int s = j & 1, qs = j % FB_QD_STAGES;  // TMEM buffer, ring stage
          // TMEM buffer s is free: the dV / dK products of chunk j - 2, which read P^T / dS^T from it, were issued
          // before this call
          if (!mbar_wait(&qd_full[qs], (uint32_t)((j / FB_QD_STAGES) & 1), abort_flag, p.status, 1220 + qs)) return false;
          tc_fence_after();
          const uint32_t q_u = qd_u + (uint32_t)qs * 2 * FB_CHUNK_BYTES, do_u = q_u + FB_CHUNK_BYTES;
#pragma unroll
          for (int kk = 0; kk < FA_D / 16; ++kk) {
            const uint32_t to = (uint32_t)(kk >> 2) * FA_BOX_BYTES, co = (uint32_t)(kk >> 2) * FB_CBOX_BYTES;
            umma_bf16_ss(tmem_base + (uint32_t)s * 128, umma_desc_kmajor_sw128(k_u + to) + 2 * (kk & 3),
                         umma_desc_kmajor_sw128(q_u + co) + 2 * (kk & 3), idesc_st, kk != 0);
          }
#pragma unroll
          for (int kk = 0; kk < FA_D / 16; ++kk) {
            const uint32_t to = (uint32_t)(kk >> 2) * FA_BOX_BYTES, co = (uint32_t)(kk >> 2) * FB_CBOX_BYTES;
            umma_bf16_ss(tmem_base + (uint32_t)s * 128 + 64, umma_desc_kmajor_sw128(v_u + to) + 2 * (kk & 3),
                         umma_desc_kmajor_sw128(do_u + co) + 2 * (kk & 3), idesc_st, kk != 0);
          }
          umma_commit(&sp_full[s]);
          return true;
        };
        if (ok) ok = issue_sp(0);
        for (int j = 0; j < n_it && ok; ++j) {
          const int s = j % FB_QD_STAGES;
          if (j + 1 < n_it) ok = issue_sp(j + 1);
          if (!ok) break;
          const int sb = j & 1;
          if (!mbar_wait(&pd_full[sb], (uint32_t)((j >> 1) & 1), abort_flag, p.status, 1240 + sb)) { ok = false; break; }
          tc_fence_after();
          const uint32_t q_u = qd_u + (uint32_t)s * 2 * FB_CHUNK_BYTES, do_u = q_u + FB_CHUNK_BYTES;
          const uint32_t pt_t = tmem_base + (uint32_t)sb * 128, dst_t = pt_t + 64;  // A operands in tensor memory
#pragma unroll
          for (int kk = 0; kk < FB_C / 16; ++kk)
            umma_bf16_ts(tmem_base + 256, pt_t + (uint32_t)kk * 8,
                         umma_desc_mnmajor_sw128(do_u + (uint32_t)kk * 2048, FB_CBOX_BYTES), idesc_acc, (j | kk) != 0);
#pragma unroll
          for (int kk = 0; kk < FB_C / 16; ++kk)
            umma_bf16_ts(tmem_base + 384, dst_t + (uint32_t)kk * 8,
                         umma_desc_mnmajor_sw128(q_u + (uint32_t)kk * 2048, FB_CBOX_BYTES), idesc_acc, (j | kk) != 0);
          umma_commit(&qd_empty[s]);
        }
        if (ok) umma_commit(acc_done);
      }
      __syncwarp();
    } else {
      const int quarter = warp & 3;
      const int r = quarter * 32 + lane;
      const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
      const int key = key_first + r;  // position inside the key segment
      const bool key_ok = key < lk;
      bool ok = true;
      for (int j = 0; j < n_it && ok; ++j) {
        const int s = j & 1;
        const int q0 = (qc_lo + j % per_head) * FB_C;
        bool full = (key_first + FA_BN <= lk) && (q0 + FB_C <= lq);
        if (p.causal) {
          full = full && (key_first + FA_BN - 1 <= q0 + off);
          if (p.window > 0) full = full && (key_first > q0 + FB_C - 1 + off - p.window);
        }
        ok = __all_sync(0xffffffffu, mbar_wait(&sp_full[s], (uint32_t)((j >> 1) & 1), abort_flag, p.status, 1250 + s));
        if (!ok) break;
        tc_fence_after();
        const float* st = stat_s + (j % FB_QD_STAGES) * 2 * FB_C;  // visible: sp_full follows the MMA that waited on qd_full
        const uint32_t ts = tmem_base + lane_off + (uint32_t)s * 128;
#pragma unroll 1
        for (int c = 0; c < FB_C; c += 32) {
          float sv[32], dp[32];
          tmem_ld_32x32(ts + c, sv);
          tmem_ld_32x32(ts + 64 + c, dp);
          tmem_ld_wait();
          if (full) {  // every key of the tile is seen by every query of the chunk
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              sv[i] = fast_exp2(fmaf(sv[i], p.scale_log2, -st[c + i]));
              dp[i] = sv[i] * ((dp[i] - st[FB_C + c + i]) * p.scale);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int qp = q0 + c + i;
              bool a = key_ok;
              if (p.causal) {
                a = a && key <= qp + off;
                if (p.window > 0) a = a && key > qp + off - p.window;
              }
              sv[i] = a ? fast_exp2(fmaf(sv[i], p.scale_log2, -st[c + i])) : 0.f;
              dp[i] = sv[i] * ((dp[i] - st[FB_C + c + i]) * p.scale);
            }
          }
          uint32_t wp[16], wd[16];  // P^T and dS^T as bf16 pairs over the columns of S^T / dP^T already read
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            wp[i] = pack_bf16(sv[2 * i], sv[2 * i + 1]);
            wd[i] = pack_bf16(dp[2 * i], dp[2 * i + 1]);
          }
          tmem_st_32x16(ts + (c >> 1), wp);
          tmem_st_32x16(ts + 64 + (c >> 1), wd);
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&pd_full[s]);
      }
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(acc_done, 0, abort_flag, p.status, 1270));
      if (ok) {
        tc_fence_after();
        __nv_bfloat16* dv = p.dv + (long long)(k_beg + key) * p.dv_rs + (long long)kvh * FA_D;
        __nv_bfloat16* dk = p.dk + (long long)(k_beg + key) * p.dk_rs + (long long)kvh * FA_D;
#pragma unroll 1
        for (int c = 0; c < FA_D; c += 32) {
          float a[32], b[32];
          tmem_ld_32x32(tmem_base + lane_off + 256 + c, a);
          tmem_ld_32x32(tmem_base + lane_off + 384 + c, b);
          tmem_ld_wait();
          if (key_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              *reinterpret_cast<uint4*>(dv + c + i) = make_uint4(pack_bf16(a[i], a[i + 1]), pack_bf16(a[i + 2], a[i + 3]),
                                                                 pack_bf16(a[i + 4], a[i + 5]), pack_bf16(a[i + 6], a[i + 7]));
              *reinterpret_cast<uint4*>(dk + c + i) = make_uint4(pack_bf16(b[i], b[i + 1]), pack_bf16(b[i + 2], b[i + 3]),
                                                                 pack_bf16(b[i + 4], b[i + 5]), pack_bf16(b[i + 6], b[i + 7]));
            }
          }
        }
        tc_fence_before();
      }
    }
  } else if (warp >= 2) {
    const int r = (warp & 3) * 32 + lane;
    const int key = key_first + r;
    if (key < lk) {
      __nv_bfloat16* dv = p.dv + (long long)(k_beg + key) * p.dv_rs + (long long)kvh * FA_D;
      __nv_bfloat16* dk = p.dk + (long long)(k_beg + key) * p.dk_rs + (long long)kvh * FA_D;
      for (int i = 0; i < FA_D; i += 8) {
        *reinterpret_cast<uint4*>(dv + i) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(dk + i) = make_uint4(0, 0, 0, 0);
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
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace trlb

// Backward of trlb_fa_varlen_fwd.  dout / out [Tq, Hq, 128], lse [Hq, Tq] from the forward; delta [Hq, Tq] fp32 is
// scratch (written here).  dq [Tq, Hq, 128], dk / dv [Tk, Hk, 128] bf16 with their own row strides.
TRLB_API int trlb_fa_varlen_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                long long q_rs, long long k_rs, long long v_rs, long long o_rs, long long do_rs,
                                const int* cu_q, const int* cu_k, int n_seq, int Tq, int Tk, int Hq, int Hk, int D,
                                float scale, int causal, int window, const float* lse, float* delta, void* dq, void* dk,
                                void* dv, long long dq_rs, long long dk_rs, long long dv_rs, int* status, cudaStream_t st) {
  if (Tq <= 0 || n_seq <= 0) return 0;
  if (D != FA_D || Hk <= 0 || Hq % Hk != 0 || (q_rs % 8) || (k_rs % 8) || (v_rs % 8) || (o_rs % 8) || (do_rs % 8) ||
      (dq_rs % 8) || (dk_rs % 8) || (dv_rs % 8))
    return -170;
  {
    const long long warps = (long long)Tq * Hq;
    const int grid = (int)((warps + 7) / 8 < 148 * 8 ? (warps + 7) / 8 : 148 * 8);
    fa_delta_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)dout, do_rs, (const __nv_bfloat16*)out, o_rs, delta, Tq, Hq);
  }
  CUtensorMap tq128, tdo128, tk64, tv64, tq64, tdo64, tk128, tv128;
  using trlb_host::make_tmap_2d_bf16;
  if (make_tmap_2d_bf16(&tq128, q, (uint64_t)Tq, (uint64_t)Hq * D, (uint64_t)q_rs, 128, 64)) return -171;
  if (make_tmap_2d_bf16(&tdo128, dout, (uint64_t)Tq, (uint64_t)Hq * D, (uint64_t)do_rs, 128, 64)) return -172;
  if (make_tmap_2d_bf16(&tk64, k, (uint64_t)Tk, (uint64_t)Hk * D, (uint64_t)k_rs, 64, 64)) return -173;
  if (make_tmap_2d_bf16(&tv64, v, (uint64_t)Tk, (uint64_t)Hk * D, (uint64_t)v_rs, 64, 64)) return -174;
  if (make_tmap_2d_bf16(&tq64, q, (uint64_t)Tq, (uint64_t)Hq * D, (uint64_t)q_rs, 64, 64)) return -175;
  if (make_tmap_2d_bf16(&tdo64, dout, (uint64_t)Tq, (uint64_t)Hq * D, (uint64_t)do_rs, 64, 64)) return -176;
  if (make_tmap_2d_bf16(&tk128, k, (uint64_t)Tk, (uint64_t)Hk * D, (uint64_t)k_rs, 128, 64)) return -177;
  if (make_tmap_2d_bf16(&tv128, v, (uint64_t)Tk, (uint64_t)Hk * D, (uint64_t)v_rs, 128, 64)) return -178;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(fa_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FA_DQ_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(fa_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FA_DKV_SMEM) != cudaSuccess)
      return -179;
    attr_set = true;
  }
  FaBwdParams p = {};
  p.cu_q = cu_q; p.cu_k = cu_k; p.n_seq = n_seq; p.Hq = Hq; p.Hk = Hk; p.causal = causal; p.window = window;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = lse; p.delta = delta; p.Tq = Tq; p.Tk = Tk;
  p.dq = (__nv_bfloat16*)dq; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
  p.dq_rs = dq_rs; p.dk_rs = dk_rs; p.dv_rs = dv_rs; p.status = status;
  const int q_tiles = (Tq + FA_BM - 1) / FA_BM + n_seq, k_tiles = (Tk + FA_BN - 1) / FA_BN + n_seq;
  fa_bwd_dkv_kernel<<<dim3(k_tiles, Hk), FA_THREADS, FA_DKV_SMEM, st>>>(tq64, tdo64, tk128, tv128, p);
  fa_bwd_dq_kernel<<<dim3(q_tiles, Hq), FA_THREADS, FA_DQ_SMEM, st>>>(tq128, tdo128, tk64, tv64, p);
  return (int)cudaGetLastError();
}
