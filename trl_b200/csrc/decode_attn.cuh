// Split-KV paged decode attention for grouped-query models (one new token per sequence).
//
// grid = (B, Hk, splits), 128 threads.  The CTA is cut into 8 groups of 16 lanes; a group owns a
// stream of tokens (4 consecutive tokens per iteration, 32 tokens per CTA iteration) and keeps its
// own online-softmax state (m, l, o) for the G = Hq/Hk query heads that share this KV head, so the
// main loop has no block-wide barrier.  A lane holds 8 of the 128 head dims: one 16-byte load of K
// and one of V per token, eight such loads in flight per lane.  Scores are reduced across the 16
// lanes with xor-shuffles.  Groups are merged through shared memory at the end and the CTA writes
// one partial (m, l, o) per head; paged_attn_combine_kernel merges the splits.
#pragma once
#include "common.cuh"

namespace trlb {

constexpr int DEC_THREADS = 128;
constexpr int MAX_G = 8;

template <int D>
__global__ void __launch_bounds__(DEC_THREADS)
paged_decode_attn_kernel(const __nv_bfloat16* __restrict__ q,  // [B, Hq, D]
                         const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                         const int* __restrict__ seq_lens, const int* __restrict__ slot_ids,
                         const int* __restrict__ block_table, int max_blocks, int block_size, int Hq, int Hk,
                         float scale, int splits, float* __restrict__ part_o,  // [B, Hq, splits, D]
                         float* __restrict__ part_ml) {                       // [B, Hq, splits, 2]
  constexpr int LPT = 16;               // lanes per token
  constexpr int DPL = D / LPT;          // dims per lane
  static_assert(DPL == 8, "one uint4 of bf16 per lane");
  constexpr int TPI = 4;                // tokens per group per iteration
  constexpr int NG = DEC_THREADS / LPT; // token groups per CTA
  constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
  const int b = blockIdx.x, kvh = blockIdx.y, sp = blockIdx.z;
  const int G = Hq / Hk;
  const int slot = slot_ids ? slot_ids[b] : b;
  const int len = seq_lens[slot] + 1;  // the new token was appended before attention
  const int tid = threadIdx.x, grp = tid / LPT, gl = tid % LPT;
  __shared__ __align__(16) float q_s[MAX_G][D];
  __shared__ float m_s[NG][MAX_G], l_s[NG][MAX_G];
  __shared__ __align__(16) float o_s[NG][MAX_G][D];

  const int per_split = ((len + splits - 1) / splits + NG * TPI - 1) / (NG * TPI) * (NG * TPI);
  const int t_begin = sp * per_split, t_end = min(len, t_begin + per_split);

  for (int i = tid; i < G * D; i += DEC_THREADS) {
    const int g = i / D, d = i % D;
    q_s[g][d] = __bfloat162float(q[((size_t)b * Hq + kvh * G + g) * D + d]) * (scale * LOG2E);
  }
  float m[MAX_G], l[MAX_G], o[MAX_G][DPL];
#pragma unroll
  for (int g = 0; g < MAX_G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int d = 0; d < DPL; ++d) o[g][d] = 0.f;
  }
  __syncthreads();
  const int* bt = block_table + (size_t)slot * max_blocks;

  // The trip count is the same for every thread of the CTA: the two token groups that share a warp
  // must reach the full-mask shuffles below together, so a group with no tokens left keeps iterating
  // on zero-filled rows and only skips the state update.
  for (int base = t_begin; base < t_end; base += NG * TPI) {
    const int t0 = base + grp * TPI;
    uint4 kraw[TPI], vraw[TPI];
#pragma unroll
    for (int k = 0; k < TPI; ++k) {
      const int tok = t0 + k;
      if (tok < t_end) {
        const int blk = bt[tok / block_size];
        const size_t row = (((size_t)blk * block_size + tok % block_size) * Hk + kvh) * D + gl * DPL;
        kraw[k] = *reinterpret_cast<const uint4*>(kc + row);
        vraw[k] = *reinterpret_cast<const uint4*>(vc + row);
      } else {
        kraw[k] = make_uint4(0, 0, 0, 0);
        vraw[k] = make_uint4(0, 0, 0, 0);
      }
    }
    float s[TPI][MAX_G];
#pragma unroll
    for (int g = 0; g < MAX_G; ++g) {
      if (g < G) {
        const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][gl * DPL]);
        const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][gl * DPL + 4]);
#pragma unroll
        for (int k = 0; k < TPI; ++k) {
          const float2 k0 = unpack_bf16(kraw[k].x), k1 = unpack_bf16(kraw[k].y), k2 = unpack_bf16(kraw[k].z),
                       k3 = unpack_bf16(kraw[k].w);
          float acc = qa.x * k0.x;
          acc = fmaf(qa.y, k0.y, acc);
          acc = fmaf(qa.z, k1.x, acc);
          acc = fmaf(qa.w, k1.y, acc);
          acc = fmaf(qb.x, k2.x, acc);
          acc = fmaf(qb.y, k2.y, acc);
          acc = fmaf(qb.z, k3.x, acc);
          acc = fmaf(qb.w, k3.y, acc);
          s[k][g] = acc;
        }
      }
    }
    // butterfly over the 16 lanes of the group: every lane ends with the full dot products
#pragma unroll
    for (int off = LPT / 2; off > 0; off >>= 1) {
#pragma unroll
      for (int g = 0; g < MAX_G; ++g) {
        if (g < G) {
#pragma unroll
          for (int k = 0; k < TPI; ++k) s[k][g] += __shfl_xor_sync(0xffffffffu, s[k][g], off);
        }
      }
    }
    float vf[TPI][DPL];
#pragma unroll
    for (int k = 0; k < TPI; ++k) {
      const float2 v0 = unpack_bf16(vraw[k].x), v1 = unpack_bf16(vraw[k].y), v2 = unpack_bf16(vraw[k].z),
                   v3 = unpack_bf16(vraw[k].w);
      vf[k][0] = v0.x; vf[k][1] = v0.y; vf[k][2] = v1.x; vf[k][3] = v1.y;
      vf[k][4] = v2.x; vf[k][5] = v2.y; vf[k][6] = v3.x; vf[k][7] = v3.y;
    }
    if (t0 >= t_end) continue;  // no shuffle or barrier below this point: safe to diverge
#pragma unroll
    for (int g = 0; g < MAX_G; ++g) {
      if (g < G) {
        float mx = s[0][g];  // token t0 is valid here
#pragma unroll
        for (int k = 1; k < TPI; ++k)
          if (t0 + k < t_end) mx = fmaxf(mx, s[k][g]);
        const float mn = fmaxf(m[g], mx);
        const float corr = exp2f(m[g] - mn);  // m = -inf on the first visit gives 0
        float p[TPI], psum = 0.f;
#pragma unroll
        for (int k = 0; k < TPI; ++k) {
          p[k] = (t0 + k < t_end) ? exp2f(s[k][g] - mn) : 0.f;
          psum += p[k];
        }
        l[g] = fmaf(l[g], corr, psum);
        m[g] = mn;
#pragma unroll
        for (int d = 0; d < DPL; ++d) {
          float acc = o[g][d] * corr;
#pragma unroll
          for (int k = 0; k < TPI; ++k) acc = fmaf(p[k], vf[k][d], acc);
          o[g][d] = acc;
        }
      }
    }
  }
  // ---- merge the token groups of this CTA ----
#pragma unroll
  for (int g = 0; g < MAX_G; ++g) {
    if (g < G) {
      *reinterpret_cast<float4*>(&o_s[grp][g][gl * DPL]) = make_float4(o[g][0], o[g][1], o[g][2], o[g][3]);
      *reinterpret_cast<float4*>(&o_s[grp][g][gl * DPL + 4]) = make_float4(o[g][4], o[g][5], o[g][6], o[g][7]);
      if (gl == 0) { m_s[grp][g] = m[g]; l_s[grp][g] = l[g]; }
    }
  }
  __syncthreads();
  for (int i = tid; i < G * D; i += DEC_THREADS) {
    const int g = i / D, d = i % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NG; ++w) M = fmaxf(M, m_s[w][g]);
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < NG; ++w) {
      const float wgt = (m_s[w][g] == -INFINITY) ? 0.f : exp2f(m_s[w][g] - M);
      acc = fmaf(o_s[w][g][d], wgt, acc);
      L = fmaf(l_s[w][g], wgt, L);
    }
    const size_t base = (((size_t)b * Hq + kvh * G + g) * splits + sp);
    part_o[base * D + d] = acc;
    if (d == 0) {
      part_ml[base * 2] = M * LN2;  // natural-log units for the combine kernel
      part_ml[base * 2 + 1] = L;
    }
  }
}

template <int D>
__global__ void paged_attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits,
                                          __nv_bfloat16* __restrict__ out, int total_heads) {
  const int h = blockIdx.x;  // b * Hq + head
  if (h >= total_heads) return;
  const int d = threadIdx.x;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[((size_t)h * splits + s) * 2]);
  float l = 0.f, o = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[((size_t)h * splits + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : __expf(ms - m);
    l += part_ml[((size_t)h * splits + s) * 2 + 1] * w;
    o += part_o[((size_t)h * splits + s) * D + d] * w;
  }
  out[(size_t)h * D + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
}

}  // namespace trlb
