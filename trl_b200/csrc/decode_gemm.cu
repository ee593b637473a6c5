// Weight-streaming GEMM for decode batches (at most 128 rows) on the 5th-generation tensor cores.
//
//     Y[b, n] = sum_k X[b, k] * W[n, k]          X [B, K] bf16, W [N, K] bf16 row-major (nn.Linear layout)
//
// With so few rows the cost is reading W once, so the kernel is laid out for bandwidth and for short launches:
//
//   * the operands are swapped: a 128-row slab of W is the M operand of tcgen05.mma, the batch (padded to 64 or
//     128) is the N operand, so no tensor-core rows are wasted on padding and the accumulator is [128 features x B];
//   * CTAs are small (a ring of 24 KB stages, under 100 KB of shared memory, 128 TMEM columns) so that two or three
//     are resident per SM: the CTAs of the NEXT kernel of the stream become resident while this one drains, and
//     their weight prefetch overlaps this kernel's epilogue (see the last point);
//   * work is cut stream-K style: the (slab, K block) steps of the whole GEMM are dealt to the resident CTAs in
//     equal contiguous runs, so every SM streams the same number of bytes whatever N is (a 28-slab projection
//     still keeps 148 SMs busy, and there is no ragged last wave);
//   * a run that does not cover a slab's whole K range adds its partial sums to an fp32 output with red.global
//     (lanes = consecutive features, one 128-byte line per warp instruction).  The consumer of that output
//     (residual add + RMSNorm, or RoPE + KV append) reads the sums and clears them, so no memset or conversion
//     kernel runs between two GEMMs;
//   * row-parallel GEMM fused with its all-reduce: with tensor-parallel peers the runs add into a LOCAL fp32
//     staging buffer and count their K blocks per (slab, 32-feature quarter); the warp whose count completes a
//     quarter reads the finished sums back from L2, clears them and adds them ONCE into the accumulator of every
//     rank (its own and, over NVLink, the peers') with 16-byte vector reductions, then bumps every rank's arrival
//     counter.  So each sum crosses NVLink once per peer whatever the stream-K split is, finished quarters go out
//     while other SMs still stream weights, and the consumer waits only on its own counter;
//   * whole-slab schedules store bf16 directly (+ bias), or apply SwiGLU: gate and up slabs of the same features go
//     to two accumulators through alternate pipeline stages and the epilogue writes silu(gate) * up;
//   * W may be stored tile-major ([slab][K block][128][64], each 16 KB tile contiguous), which turns the weight
//     stream into sequential DRAM bursts; tensor-parallel engines repack their weight slices anyway and use it;
//   * the kernel is launched with programmatic stream serialization: barrier set-up, TMEM allocation and the first
//     ring of W tiles (which do not depend on the previous kernel) are issued before griddepcontrol.wait, so the
//     ramp of each GEMM hides under the tail of the kernel before it.
//
// Stands where the reference's rollout backend (vLLM, trl/generation/vllm_generation.py:351-368,636-699) runs its
// decode linears; the reference tree itself has no such kernel.
#include "common.cuh"

namespace trlb {

constexpr int DG_BM = 128, DG_BK = 64;
constexpr int DG_THREADS = 192;
constexpr uint32_t DG_W_BYTES = DG_BM * DG_BK * 2;
constexpr int DG_MAX_PEERS = 7;

enum { DG_ACCUM_F32 = 0, DG_STORE_BF16 = 1, DG_SWIGLU = 2 };

struct DecodeGemmParams {
  int B, N, K;
  int k_blocks, slabs;
  int mode;
  int tiled;           // W is tile-major
  int steps_per_slab;  // k_blocks (x 2 with SwiGLU: gate step, up step)
  int up_slab_offset;  // SwiGLU: the up slab of features [128 j, 128 j + 128) is slab j + up_slab_offset of W
  float* Y32;          // DG_ACCUM_F32: [B, ldy] fp32, added to
  __nv_bfloat16* Yb;   // DG_STORE_BF16 / DG_SWIGLU: [B, ldy] bf16
  long long ldy;
  const __nv_bfloat16* bias;  // [N] or null (not with SwiGLU)
  int* status;
  // row-parallel all-reduce (DG_ACCUM_F32 only).  n_peers > 0: partial sums go to `stage` ([B, ldy] fp32, local,
  // zero between launches), K blocks are counted in slab_ctr[slab * 4 + quarter] (local, zero between launches) and
  // the finisher of a quarter adds the sums into Y32 and every peer_Y32 and bumps every arrive[] once.
  // n_peers == 0 with arrive[0] set: sums go straight to Y32 and every CTA bumps arrive[0] once.
  int n_peers;
  float* stage;
  uint32_t* slab_ctr;
  float* peer_Y32[DG_MAX_PEERS];
  uint32_t* arrive[DG_MAX_PEERS + 1];  // [0] = this rank's counter, then the peers'
};

template <int BN, bool SWIGLU, int STAGES>
struct DgCfg {
  static constexpr uint32_t X_BYTES = BN * DG_BK * 2;
  static constexpr uint32_t STAGE_BYTES = DG_W_BYTES + X_BYTES;
  static constexpr uint32_t ACC_COLS = SWIGLU ? 2 * BN : BN;
  static constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;  // double-buffered
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 + 256;
};

// first step and end of the run of CTA g out of G
__device__ __forceinline__ void dg_range(const DecodeGemmParams& p, int g, int G, int& u0, int& u1) {
  if (p.mode == DG_ACCUM_F32) {
    const long long total = (long long)p.slabs * p.steps_per_slab;
    u0 = (int)(total * g / G);
    u1 = (int)(total * (g + 1) / G);
  } else {  // whole slabs only: the epilogue is not additive
    u0 = (int)((long long)p.slabs * g / G) * p.steps_per_slab;
    u1 = (int)((long long)p.slabs * (g + 1) / G) * p.steps_per_slab;
  }
}

__device__ __forceinline__ void red_add_v4_sys(float* addr, const float4& v) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w) : "memory");
}
__device__ __forceinline__ void red_add_v4_gpu(float* addr, const float4& v) {
  asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w) : "memory");
}

// One warp hands the finished sums of features [f0, f0 + 32) of all B rows from the staging buffer to every rank.
// Lane l covers the float4 (l & 7) of row (l >> 3) + 4 j; four rows' loads are in flight per lane at a time.
__device__ __forceinline__ void dg_finish_quarter(const DecodeGemmParams& p, int f0, int lane) {
  const int f = f0 + 4 * (lane & 7);
  if (f < p.N) {  // N is a multiple of 4 on this path
#pragma unroll 1
    for (int rb = lane >> 3; rb < p.B; rb += 16) {
      float4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int row = rb + 4 * j;
        if (row < p.B) {
          float4* src = reinterpret_cast<float4*>(p.stage + (long long)row * p.ldy + f);
          v[j] = __ldcg(src);
          __stcg(src, make_float4(0.f, 0.f, 0.f, 0.f));
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int row = rb + 4 * j;
        if (row < p.B) {
          const long long off = (long long)row * p.ldy + f;
          red_add_v4_gpu(p.Y32 + off, v[j]);
          for (int q = 0; q < p.n_peers; ++q) red_add_v4_sys(p.peer_Y32[q] + off, v[j]);
        }
      }
    }
  }
  __threadfence_system();  // this lane's sums, before the warp's arrival below
  __syncwarp();
  if (lane == 0) {
    for (int q = 0; q <= p.n_peers; ++q)
      asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.arrive[q]) : "memory");
  }
}

template <int BN, bool SWIGLU, int STAGES, int MIN_CTAS>
__global__ void __launch_bounds__(DG_THREADS, MIN_CTAS)
decode_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   const DecodeGemmParams p) {
  using C = DgCfg<BN, SWIGLU, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::STAGE_BYTES);
  uint64_t* full_bar = bars;                     // [STAGES]
  uint64_t* empty_bar = bars + STAGES;           // [STAGES]
  uint64_t* tfull_bar = bars + 2 * STAGES;       // [2]
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int u0, u1;
  dg_range(p, (int)blockIdx.x, (int)gridDim.x, u0, u1);
  const int sps = p.steps_per_slab, kbs = p.k_blocks;

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
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();  // after the TMEM allocation, see common.cuh

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const int n_steps = u1 - u0;
      const int n_pro = n_steps < STAGES ? n_steps : STAGES;
      auto k_block = [&](int t) {
        const int s = t % sps;
        return SWIGLU ? (s >> 1) : s;
      };
      auto load_w = [&](uint8_t* sa, uint64_t* bar, int t) {
        const int s = t % sps;
        const int slab = t / sps + ((SWIGLU && (s & 1)) ? p.up_slab_offset : 0);
        const int kb = SWIGLU ? (s >> 1) : s;
        if (p.tiled) tma_load_2d(sa, &tmap_w, bar, 0, (slab * kbs + kb) * DG_BM);
        else tma_load_2d(sa, &tmap_w, bar, kb * DG_BK, slab * DG_BM);
      };
      // the first ring of weight tiles does not depend on the previous kernel
      for (int i = 0; i < n_pro; ++i) {
        mbar_expect_tx(&full_bar[i], C::STAGE_BYTES);
        load_w(smem + i * C::STAGE_BYTES, &full_bar[i], u0 + i);
      }
      pdl_wait();
      for (int i = 0; i < n_pro; ++i)
        tma_load_2d(smem + i * C::STAGE_BYTES + DG_W_BYTES, &tmap_x, &full_bar[i], k_block(u0 + i) * DG_BK, 0);
      int stage = n_pro % STAGES;
      uint32_t phase = n_pro == STAGES ? 1u : 0u;
      for (int i = n_pro; i < n_steps; ++i) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 900 + stage)) break;
        uint8_t* sa = smem + stage * C::STAGE_BYTES;
        mbar_expect_tx(&full_bar[stage], C::STAGE_BYTES);
        load_w(sa, &full_bar[stage], u0 + i);
        tma_load_2d(sa + DG_W_BYTES, &tmap_x, &full_bar[stage], k_block(u0 + i) * DG_BK, 0);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(DG_BM, BN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      int t = u0;
      while (t < u1 && ok) {
        const int s0 = t % sps;
        const int s1 = min(sps, s0 + (u1 - t));
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, 910 + acc)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tacc = tmem_base + (uint32_t)acc * C::ACC_COLS;
        for (int s = s0; s < s1; ++s) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 920 + stage)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
          const uint64_t adesc = umma_desc_kmajor_sw128(sa);
          const uint64_t bdesc = umma_desc_kmajor_sw128(sa + DG_W_BYTES);
          // SwiGLU: even steps feed the gate accumulator, odd steps the up accumulator
          const uint32_t d = SWIGLU ? tacc + (uint32_t)(s & 1) * BN : tacc;
          const uint32_t accum = (SWIGLU ? (s >= 2) : (s != s0)) ? 1u : 0u;
#pragma unroll
          for (int kk = 0; kk < DG_BK / 16; ++kk)
            umma_bf16_ss(d, adesc + 2 * kk, bdesc + 2 * kk, idesc, accum | (uint32_t)(kk != 0));
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        t += s1 - s0;
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue warps (2..5) ----------------
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    int t = u0;
    if (t < u1) pdl_wait();  // the output buffer was last touched (cleared) by an earlier kernel of the chain
    while (t < u1 && ok) {
      const int slab = t / sps, s0 = t % sps;
      const int s1 = min(sps, s0 + (u1 - t));
      const int n = slab * DG_BM + r;
      const bool n_ok = n < p.N;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, 930 + acc)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tacc = tmem_base + (uint32_t)acc * C::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
      const int c_end = min(BN, (p.B + 15) & ~15);
      float bias = 0.f;
      if (!SWIGLU && n_ok && p.bias != nullptr && s0 == 0) bias = __bfloat162float(p.bias[n]);
      // tcgen05.ld is warp-collective: the loads run for every lane, only the global writes are masked
#pragma unroll 1
      for (int c = 0; c < c_end; c += 16) {
        float v[16];
        tmem_ld_32x16(tacc + c, v);
        if (SWIGLU) {
          float u[16];
          tmem_ld_32x16(tacc + BN + c, u);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = v[i] / (1.f + __expf(-v[i])) * u[i];
        } else {
          tmem_ld_wait();
        }
        if (!n_ok) continue;
        const int rows = min(16, p.B - c);
        const long long off = (long long)c * p.ldy + n;
        if (p.mode == DG_ACCUM_F32) {
          float* dst = (p.n_peers > 0 ? p.stage : p.Y32) + off;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (i < rows) atomicAdd(dst, v[i] + bias);
            dst += p.ldy;
          }
        } else {
          __nv_bfloat16* dst = p.Yb + off;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (i < rows) *dst = __float2bfloat16(v[i] + bias);
            dst += p.ldy;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      if (p.n_peers > 0) {
        // count this run's K blocks for (slab, quarter); whoever completes the count owns the hand-over
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) {
          uint32_t* ctr = p.slab_ctr + slab * 4 + quarter;
          const uint32_t before = atomicAdd(ctr, (uint32_t)(s1 - s0));
          last = before + (uint32_t)(s1 - s0) == (uint32_t)sps;
          if (last) *ctr = 0;  // nobody else touches this word until the next launch
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          __threadfence();
          dg_finish_quarter(p, slab * DG_BM + quarter * 32, lane);
        }
      }
      t += s1 - s0;
    }
    if (p.n_peers == 0 && p.arrive[0] != nullptr) __threadfence_system();  // before the CTA's arrival below
  }
  __syncthreads();
  if (p.n_peers == 0 && p.arrive[0] != nullptr && threadIdx.x == 64) {
    __threadfence_system();
    for (int q = 0; q <= p.n_peers; ++q)
      asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.arrive[q]) : "memory");
  }
  if (*abort_flag) {
    // a role gave up: let copies in flight land before the shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// dst tile-major <- src row-major [rows, K] (row stride lds); rows / columns beyond the source become zeros.
// One 16-byte vector per thread; a tile is [128][64] bf16 = 1024 vectors.
__global__ void __launch_bounds__(256) tile_weights_kernel(const __nv_bfloat16* __restrict__ src, long long lds,
                                                           __nv_bfloat16* __restrict__ dst, int rows, int K,
                                                           int k_blocks, long long n_vec) {
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < n_vec; v += (long long)gridDim.x * blockDim.x) {
    const long long tile = v >> 10;
    const int in_tile = (int)(v & 1023), r = in_tile >> 3, c8 = in_tile & 7;
    const int slab = (int)(tile / k_blocks), kb = (int)(tile % k_blocks);
    const int row = slab * DG_BM + r, col = kb * DG_BK + c8 * 8;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (row < rows && col < K) val = *reinterpret_cast<const uint4*>(src + (long long)row * lds + col);  // K % 8 == 0
    reinterpret_cast<uint4*>(dst)[v] = val;
  }
}

}  // namespace trlb

using namespace trlb;

namespace {

int g_ctas_per_sm = 2;  // 64-row variants: 2 (4-stage ring) or 3 (3-stage ring); set by trlb_decode_gemm_set_ctas_per_sm

template <int BN, bool SWIGLU, int STAGES, int MIN_CTAS>
int dg_launch(const CUtensorMap& tw, const CUtensorMap& tx, const DecodeGemmParams& p, int ctas, cudaStream_t st) {
  using C = DgCfg<BN, SWIGLU, STAGES>;
  auto kern = decode_gemm_kernel<BN, SWIGLU, STAGES, MIN_CTAS>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM) != cudaSuccess) return -153;
    attr_set = true;
  }
  return (int)trlb_host::launch_kernel(kern, dim3(ctas), dim3(DG_THREADS), C::SMEM, st, trlb_host::pdl_enabled(), tw, tx, p);
}

int dg_ctas_per_sm(int B, int mode) {
  if (B > 64) return (mode == DG_SWIGLU || g_ctas_per_sm < 2) ? 1 : 2;  // 128-row tiles: 256 / 512 TMEM columns each
  if (mode == DG_SWIGLU) return 1;  // SwiGLU slabs cannot be split along K: one CTA per SM with a deep ring
  return g_ctas_per_sm;
}

}  // namespace

// Resident CTAs per SM for batches of at most 64 rows: 2 (default; 4-stage rings) or 3 (3-stage rings).  Returns
// the previous value.  More, smaller CTAs let more of the next kernel's weight prefetch overlap this kernel's tail.
TRLB_API int trlb_decode_gemm_set_ctas_per_sm(int n) {
  const int was = g_ctas_per_sm;
  if (n >= 1 && n <= 3) g_ctas_per_sm = n;
  return was;
}

// Number of CTAs trlb_decode_gemm launches for this problem (the arrival count a consumer of the fused all-reduce
// waits for is ranks x this).
TRLB_API int trlb_decode_gemm_ctas(int B, int N, int K, int mode, int max_ctas) {
  const int k_blocks = (K + DG_BK - 1) / DG_BK;
  const int slabs = (N + DG_BM - 1) / DG_BM;
  int ctas = trlb_host::sm_count() * dg_ctas_per_sm(B, mode);
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  if (mode == DG_ACCUM_F32) {
    const long long total = (long long)slabs * k_blocks;
    const long long cap = total / 4 > 0 ? total / 4 : 1;  // at least 4 K blocks per CTA
    if (ctas > cap) ctas = (int)cap;
  } else if (ctas > slabs) {
    ctas = slabs;
  }
  return ctas;
}

// Arrivals per rank of one fused all-reduce GEMM with N output features (one per slab and 32-feature quarter).
TRLB_API int trlb_decode_gemm_arrivals(int N) { return 4 * ((N + DG_BM - 1) / DG_BM); }

// X [B, K] bf16 (row stride ldx), B <= 128.  W bf16: row-major with row stride ldw, or (tiled != 0) tile-major
// [ceil(rows/128)][ceil(K/64)][128][64] as written by trlb_tile_weights.
//   mode 0  W [N, K];  Y32 [B, N] fp32 (row stride ldy) is added to (+ bias once): the caller provides zeros
//   mode 1  W [N, K];  Yb  [B, N] bf16 = X W^T (+ bias)
//   mode 2  W [2N, K] (gate rows, then up rows; N a multiple of 128);  Yb [B, N] bf16 = silu(X Wg^T) * (X Wu^T)
// max_ctas: 0 = every SM with its resident CTAs, else an upper bound on the grid.
// Fused all-reduce (mode 0, n_peers > 0): peer_y32[i] is the same buffer on peer i; arrive[0] is this rank's arrival
// counter and arrive[1 + i] peer i's; stage is a local zeroed fp32 buffer shaped like Y32 and slab_ctr a local zeroed
// array of 4 * ceil(N / 128) words (both are left zeroed); N and ldy multiples of 4.  Every (slab, quarter) adds 1
// to every counter once its sums are visible system-wide: a consumer waits for ranks * trlb_decode_gemm_arrivals(N).
// arrive may also be given with n_peers == 0: then each CTA adds 1 to arrive[0] (trlb_decode_gemm_ctas of them).
TRLB_API int trlb_decode_gemm(const void* X, const void* W, const void* bias, float* Y32, void* Yb, int B, int N, int K,
                              long long ldx, long long ldw, long long ldy, int mode, int tiled, int max_ctas, int n_peers,
                              float* const* peer_y32, uint32_t* const* arrive, float* stage, uint32_t* slab_ctr,
                              int* status, cudaStream_t st) {
  if (B <= 0 || N <= 0 || K <= 0) return 0;
  if (B > 128 || (K % 8) != 0 || (ldx % 8) != 0 || mode < 0 || mode > 2) return -150;
  if (!tiled && (ldw % 8) != 0) return -150;
  if (mode == DG_SWIGLU && (bias != nullptr || (N % DG_BM) != 0)) return -150;
  if (n_peers < 0 || n_peers > DG_MAX_PEERS || (n_peers > 0 && (mode != DG_ACCUM_F32 || !peer_y32 || !arrive))) return -150;
  if (n_peers > 0 && (!stage || !slab_ctr || (N % 4) != 0 || (ldy % 4) != 0 || (reinterpret_cast<uintptr_t>(Y32) & 15) ||
                      (reinterpret_cast<uintptr_t>(stage) & 15)))
    return -150;
  const int BN = B <= 64 ? 64 : 128;
  const long long w_rows = mode == DG_SWIGLU ? 2LL * N : N;
  DecodeGemmParams p = {};
  p.B = B; p.N = N; p.K = K; p.mode = mode; p.tiled = tiled ? 1 : 0;
  p.k_blocks = (K + DG_BK - 1) / DG_BK;
  p.slabs = (N + DG_BM - 1) / DG_BM;
  p.steps_per_slab = p.k_blocks * (mode == DG_SWIGLU ? 2 : 1);
  p.up_slab_offset = p.slabs;
  CUtensorMap tw, tx;
  if (tiled) {
    const uint64_t tiles = (uint64_t)((w_rows + DG_BM - 1) / DG_BM) * p.k_blocks;
    if (trlb_host::make_tmap_2d_bf16(&tw, W, tiles * DG_BM, DG_BK, DG_BK, DG_BM, DG_BK)) return -151;
  } else if (trlb_host::make_tmap_2d_bf16(&tw, W, (uint64_t)w_rows, (uint64_t)K, (uint64_t)ldw, DG_BM, DG_BK)) {
    return -151;
  }
  if (trlb_host::make_tmap_2d_bf16(&tx, X, (uint64_t)B, (uint64_t)K, (uint64_t)ldx, (uint32_t)BN, DG_BK)) return -152;
  p.Y32 = Y32; p.Yb = (__nv_bfloat16*)Yb; p.ldy = ldy; p.bias = (const __nv_bfloat16*)bias; p.status = status;
  p.n_peers = n_peers; p.stage = stage; p.slab_ctr = slab_ctr;
  if (arrive != nullptr && mode == DG_ACCUM_F32) p.arrive[0] = arrive[0];
  for (int i = 0; i < n_peers; ++i) { p.peer_Y32[i] = peer_y32[i]; p.arrive[1 + i] = arrive[1 + i]; }
  const int ctas = trlb_decode_gemm_ctas(B, N, K, mode, max_ctas);
  if (BN == 64) {
    if (mode == DG_SWIGLU) return dg_launch<64, true, 8, 1>(tw, tx, p, ctas, st);
    if (g_ctas_per_sm == 3) return dg_launch<64, false, 3, 3>(tw, tx, p, ctas, st);
    return dg_launch<64, false, 4, 2>(tw, tx, p, ctas, st);
  }
  if (mode == DG_SWIGLU) return dg_launch<128, true, 6, 1>(tw, tx, p, ctas, st);
  if (g_ctas_per_sm < 2) return dg_launch<128, false, 6, 1>(tw, tx, p, ctas, st);
  return dg_launch<128, false, 3, 2>(tw, tx, p, ctas, st);
}

// Number of bf16 elements of the tile-major copy of a [rows, K] weight.
TRLB_API long long trlb_tiled_elems(int rows, int K) {
  return (long long)((rows + DG_BM - 1) / DG_BM) * ((K + DG_BK - 1) / DG_BK) * DG_BM * DG_BK;
}

// dst (trlb_tiled_elems(rows, K) bf16) <- tile-major copy of src [rows, K] (row stride lds; K and lds multiples of 8,
// both pointers 16-byte aligned).
TRLB_API int trlb_tile_weights(const void* src, long long lds, void* dst, int rows, int K, cudaStream_t st) {
  if (rows <= 0 || K <= 0) return 0;
  if ((lds % 8) != 0 || (K % 8) != 0 || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15))
    return -154;
  const int k_blocks = (K + DG_BK - 1) / DG_BK;
  const long long n_vec = trlb_tiled_elems(rows, K) / 8;
  const long long want = (n_vec + 255) / 256;
  const int grid = (int)(want < 148 * 16 ? want : 148 * 16);
  tile_weights_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)src, lds, (__nv_bfloat16*)dst, rows, K, k_blocks, n_vec);
  return (int)cudaGetLastError();
}
