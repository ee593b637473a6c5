// Rollout-engine decode kernels (one new token per running sequence):
//
//  rope_kv_write      RoPE on q and k of the fused QKV row, k/v appended to the paged cache
//  kv_write_prefill   k/v of a packed prefill written to the paged cache
//  paged_decode_attn  split-KV attention of 1 query token against the paged cache (GQA)
//  sample_tokens      temperature / min-p / EOS-probability-floor sampling by Gumbel-max with
//                     the sampled token's log-probability in the processed distribution
//
// They stand where the reference uses vLLM's CUDA kernels (trl/generation/vllm_generation.py:351-368,680).
#include "common.cuh"
#include "decode_attn.cuh"

namespace trlb {

// ------------------------------------------------------------------------------------------
// cache layout: K and V are [num_blocks, block_size, Hk, D] bf16; block_table [max_seqs, max_blocks]
// ------------------------------------------------------------------------------------------
__global__ void rope_kv_write_kernel(const __nv_bfloat16* __restrict__ qkv, long long row_stride,
                                     const int* __restrict__ seq_lens, const int* __restrict__ slot_ids,
                                     const int* __restrict__ block_table, int max_blocks, int block_size,
                                     __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ kc,
                                     __nv_bfloat16* __restrict__ vc, int B, int Hq, int Hk, int D, float log2_theta,
                                     int v_t, const int* __restrict__ pos_delta) {
  const int half = D >> 1;
  const int per_tok = (Hq + 2 * Hk) * half;
  const long long total = (long long)B * per_tok;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(idx / per_tok);
    int r = (int)(idx % per_tok);
    const int head = r / half, f = r % half;
    const int slot = slot_ids ? slot_ids[b] : b;
    const int pos = seq_lens[slot];  // position of the new token = current length
    if (pos < 0) continue;            // inactive slot
    const __nv_bfloat16* src = qkv + (size_t)b * row_stride + (size_t)head * D;
    const int blk = block_table[(size_t)slot * max_blocks + pos / block_size];
    const size_t cache_row = ((size_t)blk * block_size + pos % block_size) * Hk;
    if (head < Hq + Hk) {
      const float inv = exp2f(-log2_theta * (float)(2 * f) / (float)D);
      float s, c;
      sincosf((float)(pos + (pos_delta ? pos_delta[slot] : 0)) * inv, &s, &c);  // rotary position may lead the cache slot
      const float lo = __bfloat162float(src[f]), hi = __bfloat162float(src[half + f]);
      const float o0 = lo * c - hi * s, o1 = hi * c + lo * s;
      __nv_bfloat16* dst = head < Hq ? q_out + ((size_t)b * Hq + head) * D : kc + (cache_row + (head - Hq)) * D;
      dst[f] = __float2bfloat16(o0);
      dst[half + f] = __float2bfloat16(o1);
    } else if (v_t) {
      // V transposed inside the page: [block, head, dim, token]
      __nv_bfloat16* dst = vc + (((size_t)blk * Hk + (head - Hq - Hk)) * D) * block_size + pos % block_size;
      dst[(size_t)f * block_size] = src[f];
      dst[(size_t)(half + f) * block_size] = src[half + f];
    } else {
      __nv_bfloat16* dst = vc + (cache_row + (head - Hq - Hk)) * D;
      dst[f] = src[f];
      dst[half + f] = src[half + f];
    }
  }
}

// Variant fed by the stream-K decode GEMM: the fused QKV row arrives as fp32 partial sums, which are consumed
// (bias added, optional per-head RMSNorm of q and k as in Qwen3, RoPE, cache append) and cleared here, so the next
// step's GEMM accumulates from zero without a memset.  One warp per (token, head); each lane owns the rotation pairs
// (f, f + D/2) for f = lane, lane + 32, ...
__global__ void __launch_bounds__(256)
rope_kv_write_f32_kernel(float* __restrict__ acc, long long row_stride, const __nv_bfloat16* __restrict__ bias,
                         const __nv_bfloat16* __restrict__ q_norm, const __nv_bfloat16* __restrict__ k_norm,
                         float norm_eps, const int* __restrict__ seq_lens, const int* __restrict__ slot_ids,
                         const int* __restrict__ block_table, int max_blocks, int block_size,
                         __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc,
                         int B, int Hq, int Hk, int D, float log2_theta, int v_t, const int* __restrict__ pos_delta) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = D >> 1, heads = Hq + 2 * Hk;
  const int lane = threadIdx.x & 31;
  const int warps_total = (gridDim.x * blockDim.x) >> 5;
  for (int item = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; item < B * heads; item += warps_total) {
    const int b = item / heads, head = item % heads;
    const int slot = slot_ids ? slot_ids[b] : b;
    const int pos = seq_lens[slot];
    float* src = acc + (size_t)b * row_stride + (size_t)head * D;
    const __nv_bfloat16* bsrc = bias ? bias + (size_t)head * D : nullptr;
    float lo[2], hi[2];  // D <= 128: at most two pairs per lane
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int f = lane + 32 * j;
      lo[j] = hi[j] = 0.f;
      if (f < half) {
        lo[j] = src[f];
        hi[j] = src[half + f];
        src[f] = 0.f;
        src[half + f] = 0.f;
        if (bsrc) { lo[j] += __bfloat162float(bsrc[f]); hi[j] += __bfloat162float(bsrc[half + f]); }
        // from here on the projection has the precision of the unfused path (a bf16 GEMM output)
        lo[j] = __bfloat162float(__float2bfloat16(lo[j]));
        hi[j] = __bfloat162float(__float2bfloat16(hi[j]));
        ss += lo[j] * lo[j] + hi[j] * hi[j];
      }
    }
    if (pos < 0) continue;  // inactive slot: sums are dropped
    const __nv_bfloat16* nw = head < Hq ? q_norm : (head < Hq + Hk ? k_norm : nullptr);
    if (nw != nullptr) {
      const float rstd = rsqrtf(warp_sum(ss) / (float)D + norm_eps);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int f = lane + 32 * j;
        if (f < half) {
          // the normalised value is rounded to bf16 before the rotation, as the unfused path does
          lo[j] = __bfloat162float(__float2bfloat16(lo[j] * rstd * __bfloat162float(nw[f])));
          hi[j] = __bfloat162float(__float2bfloat16(hi[j] * rstd * __bfloat162float(nw[half + f])));
        }
      }
    }
    const int blk = block_table[(size_t)slot * max_blocks + pos / block_size];
    const size_t cache_row = ((size_t)blk * block_size + pos % block_size) * Hk;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int f = lane + 32 * j;
      if (f >= half) continue;
      if (head < Hq + Hk) {
        const float l = lo[j], h = hi[j];
        const float inv = exp2f(-log2_theta * (float)(2 * f) / (float)D);
        float sn, cs;
        sincosf((float)(pos + (pos_delta ? pos_delta[slot] : 0)) * inv, &sn, &cs);
        __nv_bfloat16* dst = head < Hq ? q_out + ((size_t)b * Hq + head) * D : kc + (cache_row + (head - Hq)) * D;
        dst[f] = __float2bfloat16(l * cs - h * sn);
        dst[half + f] = __float2bfloat16(h * cs + l * sn);
      } else if (v_t) {
        __nv_bfloat16* dst = vc + (((size_t)blk * Hk + (head - Hq - Hk)) * D) * block_size + pos % block_size;
        dst[(size_t)f * block_size] = __float2bfloat16(lo[j]);
        dst[(size_t)(half + f) * block_size] = __float2bfloat16(hi[j]);
      } else {
        __nv_bfloat16* dst = vc + (cache_row + (head - Hq - Hk)) * D;
        dst[f] = __float2bfloat16(lo[j]);
        dst[half + f] = __float2bfloat16(hi[j]);
      }
    }
  }
}

// Same consumer without the per-head norm: one thread per rotation pair, laid out like rope_kv_write_kernel.
__global__ void __launch_bounds__(256)
rope_kv_write_f32_flat_kernel(float* __restrict__ acc, long long row_stride, const __nv_bfloat16* __restrict__ bias,
                              const int* __restrict__ seq_lens, const int* __restrict__ slot_ids,
                              const int* __restrict__ block_table, int max_blocks, int block_size,
                              __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ kc,
                              __nv_bfloat16* __restrict__ vc, int B, int Hq, int Hk, int D, float log2_theta, int v_t,
                              const int* __restrict__ pos_delta) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = D >> 1;
  const int per_tok = (Hq + 2 * Hk) * half;
  const long long total = (long long)B * per_tok;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(idx / per_tok);
    const int r = (int)(idx % per_tok);
    const int head = r / half, f = r % half;
    float* src = acc + (size_t)b * row_stride + (size_t)head * D;
    float lo = src[f], hi = src[half + f];
    src[f] = 0.f;
    src[half + f] = 0.f;
    const int slot = slot_ids ? slot_ids[b] : b;
    const int pos = seq_lens[slot];
    if (pos < 0) continue;  // inactive slot: the sums are dropped
    if (bias != nullptr) {
      lo += __bfloat162float(bias[(size_t)head * D + f]);
      hi += __bfloat162float(bias[(size_t)head * D + half + f]);
    }
    lo = __bfloat162float(__float2bfloat16(lo));  // the precision of a bf16 GEMM output
    hi = __bfloat162float(__float2bfloat16(hi));
    const int blk = block_table[(size_t)slot * max_blocks + pos / block_size];
    const size_t cache_row = ((size_t)blk * block_size + pos % block_size) * Hk;
    if (head < Hq + Hk) {
      const float inv = exp2f(-log2_theta * (float)(2 * f) / (float)D);
      float sn, cs;
      sincosf((float)(pos + (pos_delta ? pos_delta[slot] : 0)) * inv, &sn, &cs);
      __nv_bfloat16* dst = head < Hq ? q_out + ((size_t)b * Hq + head) * D : kc + (cache_row + (head - Hq)) * D;
      dst[f] = __float2bfloat16(lo * cs - hi * sn);
      dst[half + f] = __float2bfloat16(hi * cs + lo * sn);
    } else if (v_t) {
      __nv_bfloat16* dst = vc + (((size_t)blk * Hk + (head - Hq - Hk)) * D) * block_size + pos % block_size;
      dst[(size_t)f * block_size] = __float2bfloat16(lo);
      dst[(size_t)(half + f) * block_size] = __float2bfloat16(hi);
    } else {
      __nv_bfloat16* dst = vc + (cache_row + (head - Hq - Hk)) * D;
      dst[f] = __float2bfloat16(lo);
      dst[half + f] = __float2bfloat16(hi);
    }
  }
}

// k,v [T,Hk,D] (already rotated) of packed prompts -> cache.  tok_slot[t], tok_pos[t] give the
// destination sequence slot and position of token t.
__global__ void kv_write_prefill_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                        long long k_stride, long long v_stride, const int* __restrict__ tok_slot,
                                        const int* __restrict__ tok_pos, const int* __restrict__ block_table,
                                        int max_blocks, int block_size, __nv_bfloat16* __restrict__ kc,
                                        __nv_bfloat16* __restrict__ vc, int T, int Hk, int D, int v_t) {
  const int vec_per_tok = Hk * D / 8;
  const long long total = (long long)T * vec_per_tok;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / vec_per_tok), e = (int)(idx % vec_per_tok);
    const int slot = tok_slot[t], pos = tok_pos[t];
    if (slot < 0) continue;
    const int blk = block_table[(size_t)slot * max_blocks + pos / block_size];
    const size_t row = ((size_t)blk * block_size + pos % block_size) * Hk * D;
    reinterpret_cast<uint4*>(kc + row)[e] = reinterpret_cast<const uint4*>(k + (size_t)t * k_stride)[e];
    if (!v_t) {
      reinterpret_cast<uint4*>(vc + row)[e] = reinterpret_cast<const uint4*>(v + (size_t)t * v_stride)[e];
    } else {
      const uint4 u = reinterpret_cast<const uint4*>(v + (size_t)t * v_stride)[e];
      const __nv_bfloat16* vals = reinterpret_cast<const __nv_bfloat16*>(&u);
      const int h = (e * 8) / D, d0 = (e * 8) % D;
      __nv_bfloat16* dst = vc + (((size_t)blk * Hk + h) * D + d0) * block_size + pos % block_size;
#pragma unroll
      for (int i = 0; i < 8; ++i) dst[(size_t)i * block_size] = vals[i];
    }
  }
}

// ------------------------------------------------------------------------------------------
// Sampler.  One CTA per row.  Pass 1: max and log-sum-exp of the processed logits without the
// EOS column.  Pass 2: Gumbel-max over the final distribution.  Outputs token id and its log-prob.
// Processing order: repetition handled by caller; temperature; min-p; EOS probability floor.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t hash_u32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ float uniform01(uint32_t seed, uint32_t step, uint32_t row, uint32_t col) {
  uint32_t h = hash_u32(seed ^ hash_u32(step * 0x9E3779B9U + row) ^ hash_u32(col * 0x85EBCA6BU + 0x165667B1U));
  h = hash_u32(h + col);
  return ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

template <typename T>
__device__ __forceinline__ float ld_logit(const T* p, long long i);
template <>
__device__ __forceinline__ float ld_logit<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}

template <typename T>
__global__ void __launch_bounds__(1024)
sample_kernel(const T* __restrict__ logits, long long row_stride, int V, float inv_temp, float min_p, int eos_id,
              float eos_floor, uint32_t seed, const int* __restrict__ step_ptr, int greedy,
              int* __restrict__ out_tok, float* __restrict__ out_logp) {
  const int row = blockIdx.x;
  const T* z = logits + (size_t)row * row_stride;
  __shared__ float sh_a[32], sh_b[32];
  __shared__ int sh_i[32];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
  const uint32_t step = step_ptr ? (uint32_t)(*step_ptr) : 0u;
  // pass 1: max over all, then sum-exp excluding eos
  float mx = -INFINITY;
  for (int i = tid; i < V; i += blockDim.x) mx = fmaxf(mx, ld_logit<T>(z, i) * inv_temp);
  mx = warp_max(mx);
  if (lane == 0) sh_a[wid] = mx;
  __syncthreads();
  mx = -INFINITY;
  for (int w = 0; w < nw; ++w) mx = fmaxf(mx, sh_a[w]);
  __syncthreads();
  const float thresh = (min_p > 0.f) ? mx + __logf(min_p) : -INFINITY;  // keep p >= min_p * p_max
  float se = 0.f;
  for (int i = tid; i < V; i += blockDim.x) {
    const float v = ld_logit<T>(z, i) * inv_temp;
    if (i != eos_id && v >= thresh) se += __expf(v - mx);
  }
  se = warp_sum(se);
  if (lane == 0) sh_a[wid] = se;
  __syncthreads();
  se = 0.f;
  for (int w = 0; w < nw; ++w) se += sh_a[w];
  __syncthreads();
  // eos handling
  float z_eos = -INFINITY;
  if (eos_id >= 0 && eos_id < V) {
    z_eos = ld_logit<T>(z, eos_id) * inv_temp;
    if (z_eos < thresh) z_eos = -INFINITY;
  }
  const float lse_others = mx + __logf(fmaxf(se, 1e-30f));
  float lse_all;
  if (eos_floor > 0.f && eos_id >= 0) {
    // p(eos) = max(p(eos), floor): raise the eos logit until softmax gives the floor
    const float need = lse_others + __logf(eos_floor / (1.f - eos_floor));
    if (z_eos < need) z_eos = need;
  }
  {
    const float a = fmaxf(lse_others, z_eos);
    lse_all = a + __logf(__expf(lse_others - a) + __expf(z_eos - a));
  }
  // pass 2: Gumbel-max (or plain argmax when greedy)
  float best = -INFINITY;
  int best_i = 0;
  float best_z = 0.f;
  for (int i = tid; i < V; i += blockDim.x) {
    float v = (i == eos_id) ? z_eos : ld_logit<T>(z, i) * inv_temp;
    if (v < thresh && i != eos_id) continue;
    if (v == -INFINITY) continue;
    float key = v;
    if (!greedy) {
      const float u = uniform01(seed, step, (uint32_t)row, (uint32_t)i);
      key = v - __logf(-__logf(u));
    }
    if (key > best) { best = key; best_i = i; best_z = v; }
  }
  // block arg-max
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    const float oz = __shfl_xor_sync(0xffffffffu, best_z, o);
    if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; best_z = oz; }
  }
  if (lane == 0) { sh_a[wid] = best; sh_i[wid] = best_i; sh_b[wid] = best_z; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < nw; ++w)
      if (sh_a[w] > best || (sh_a[w] == best && sh_i[w] < best_i)) { best = sh_a[w]; best_i = sh_i[w]; best_z = sh_b[w]; }
    out_tok[row] = best_i;
    out_logp[row] = best_z - lse_all;
  }
}

// Single-pass sampler for the common case (bf16 logits, no min-p): gridDim.y CTAs share a row, each keeps an
// online (max, sum-exp) and its Gumbel-max candidate over its slice of the vocabulary; the CTA that arrives
// last on the row's counter merges the partials, applies the EOS floor, scores the EOS column and writes the
// token and its log-prob.  The counter is left at zero for the next call.
__device__ __forceinline__ float uniform01_pre(uint32_t base, uint32_t col) {
  uint32_t h = hash_u32(base ^ hash_u32(col * 0x85EBCA6BU + 0x165667B1U));
  h = hash_u32(h + col);
  return ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(512)
sample_split_kernel(const __nv_bfloat16* __restrict__ logits, long long row_stride, int V, float inv_temp, int eos_id,
                    float eos_floor, uint32_t seed, const int* __restrict__ step_ptr, int greedy,
                    float4* __restrict__ part, int* __restrict__ part_i, unsigned* __restrict__ counter,
                    int* __restrict__ out_tok, float* __restrict__ out_logp) {
  const int row = blockIdx.x, sp = blockIdx.y, S = gridDim.y;
  const __nv_bfloat16* z = logits + (size_t)row * row_stride;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
  const uint32_t step = step_ptr ? (uint32_t)(*step_ptr) : 0u;
  const uint32_t base = seed ^ hash_u32(step * 0x9E3779B9U + (uint32_t)row);
  const int nvec = V >> 3, per = (nvec + S - 1) / S;
  const int v0 = sp * per, v1 = min(nvec, v0 + per);
  float m = -INFINITY, se = 0.f, best = -INFINITY, best_z = 0.f;
  int best_i = -1;
  for (int i = v0 + tid; i < v1; i += blockDim.x) {
    const uint4 u = reinterpret_cast<const uint4*>(z)[i];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float2 f = unpack_bf16(w[k >> 1]);
      const float x = ((k & 1) ? f.y : f.x) * inv_temp;
      const int col = i * 8 + k;
      if (col == eos_id || x == -INFINITY) continue;
      if (x > m) { se = se * __expf(m - x) + 1.f; m = x; } else { se += __expf(x - m); }
      const float key = greedy ? x : x - __logf(-__logf(uniform01_pre(base, (uint32_t)col)));
      if (key > best) { best = key; best_i = col; best_z = x; }
    }
  }
  // block reduction
  __shared__ float sh_m[16], sh_s[16], sh_b[16], sh_z[16];
  __shared__ int sh_i[16];
  __shared__ int is_last;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, se, o);
    const float nm = fmaxf(m, om);
    se = (nm == -INFINITY) ? 0.f : se * __expf(m - nm) + os * __expf(om - nm);
    m = nm;
    const float ob = __shfl_xor_sync(0xffffffffu, best, o), oz = __shfl_xor_sync(0xffffffffu, best_z, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi >= 0 && (best_i < 0 || oi < best_i))) { best = ob; best_i = oi; best_z = oz; }
  }
  if (lane == 0) { sh_m[wid] = m; sh_s[wid] = se; sh_b[wid] = best; sh_z[wid] = best_z; sh_i[wid] = best_i; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < nw; ++w) {
      const float nm = fmaxf(m, sh_m[w]);
      se = (nm == -INFINITY) ? 0.f : se * __expf(m - nm) + sh_s[w] * __expf(sh_m[w] - nm);
      m = nm;
      if (sh_b[w] > best || (sh_b[w] == best && sh_i[w] >= 0 && (best_i < 0 || sh_i[w] < best_i))) {
        best = sh_b[w]; best_i = sh_i[w]; best_z = sh_z[w];
      }
    }
    part[(size_t)row * 8 + sp] = make_float4(m, se, best, best_z);
    part_i[(size_t)row * 8 + sp] = best_i;
    __threadfence();
    is_last = (atomicAdd(&counter[row], 1u) == (unsigned)(S - 1));
    if (is_last) {
      __threadfence();
      float M = -INFINITY;
      for (int q = 0; q < S; ++q) M = fmaxf(M, __ldcg(&part[(size_t)row * 8 + q]).x);
      float tot = 0.f;
      best = -INFINITY; best_i = -1; best_z = 0.f;
      for (int q = 0; q < S; ++q) {
        const float4 pq = __ldcg(&part[(size_t)row * 8 + q]);
        const int pi = __ldcg(&part_i[(size_t)row * 8 + q]);
        if (pq.x != -INFINITY) tot += pq.y * __expf(pq.x - M);
        if (pi >= 0 && (pq.z > best || (pq.z == best && (best_i < 0 || pi < best_i)))) { best = pq.z; best_i = pi; best_z = pq.w; }
      }
      const float lse_others = M + __logf(fmaxf(tot, 1e-30f));
      float z_eos = -INFINITY;
      if (eos_id >= 0 && eos_id < V) z_eos = __bfloat162float(z[eos_id]) * inv_temp;
      if (eos_floor > 0.f && eos_id >= 0 && eos_id < V) {
        const float need = lse_others + __logf(eos_floor / (1.f - eos_floor));
        if (z_eos < need) z_eos = need;
      }
      const float a = fmaxf(lse_others, z_eos);
      const float lse_all = a + __logf(__expf(lse_others - a) + __expf(z_eos - a));
      if (z_eos != -INFINITY) {
        const float key = greedy ? z_eos : z_eos - __logf(-__logf(uniform01_pre(base, (uint32_t)eos_id)));
        if (key > best || (key == best && eos_id < best_i) || best_i < 0) { best = key; best_i = eos_id; best_z = z_eos; }
      }
      out_tok[row] = best_i < 0 ? 0 : best_i;
      out_logp[row] = best_z - lse_all;
      counter[row] = 0;
    }
  }
}

// After sampling: append token to the output buffer, bump lengths, mark finished sequences.
// out_tokens / out_logps are [max_seqs, max_new]; n_gen[slot] counts generated tokens.
__global__ void advance_kernel(const int* __restrict__ tok, const float* __restrict__ logp, const int* __restrict__ slot_ids,
                               int B, int* __restrict__ seq_lens, int* __restrict__ n_gen, int* __restrict__ finished,
                               int* __restrict__ out_tokens, float* __restrict__ out_logps, int max_new, int eos_id,
                               int max_total_len, long long* __restrict__ next_input, int* __restrict__ step_counter,
                               int bump_len) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b == 0 && step_counter) atomicAdd(step_counter, 1);
  if (b >= B) return;
  const int slot = slot_ids ? slot_ids[b] : b;
  if (seq_lens[slot] < 0) return;
  if (finished[slot]) { next_input[b] = eos_id >= 0 ? eos_id : 0; return; }
  const int t = tok[b];
  const int g = n_gen[slot];
  if (g < max_new) {
    out_tokens[(size_t)slot * max_new + g] = t;
    out_logps[(size_t)slot * max_new + g] = logp[b];
  }
  n_gen[slot] = g + 1;
  seq_lens[slot] += bump_len;  // decode: the token whose K/V was just written now counts
  next_input[b] = t;
  if (t == eos_id || g + 1 >= max_new || seq_lens[slot] + 1 >= max_total_len) {
    finished[slot] = 1;
    // a finished slot stops costing KV traffic at once: negative length = inactive for the
    // RoPE/KV-append and attention kernels (the host reads n_gen and the output rows, not seq_lens)
    seq_lens[slot] = -1;
  }
}

}  // namespace trlb

using namespace trlb;

TRLB_API int trlb_rope_kv_write(const void* qkv, long long row_stride, const int* seq_lens, const int* slot_ids,
                                const int* block_table, int max_blocks, int block_size, void* q_out, void* kc, void* vc,
                                int B, int Hq, int Hk, int D, float theta, int v_t, const int* pos_delta,
                                cudaStream_t st) {
  if (B == 0) return 0;
  const long long work = (long long)B * (Hq + 2 * Hk) * (D / 2);
  int grid = (int)((work + 255) / 256);
  rope_kv_write_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)qkv, row_stride, seq_lens, slot_ids, block_table,
                                             max_blocks, block_size, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kc,
                                             (__nv_bfloat16*)vc, B, Hq, Hk, D, log2f(theta), v_t, pos_delta);
  return (int)cudaGetLastError();
}

// fp32 sums in, cleared on the way (see rope_kv_write_f32_kernel).  bias / q_norm / k_norm may be null.  D <= 128.
TRLB_API int trlb_rope_kv_write_f32(float* acc, long long row_stride, const void* bias, const void* q_norm,
                                    const void* k_norm, float norm_eps, const int* seq_lens, const int* slot_ids,
                                    const int* block_table, int max_blocks, int block_size, void* q_out, void* kc,
                                    void* vc, int B, int Hq, int Hk, int D, float theta, int v_t,
                                    const int* pos_delta, cudaStream_t st) {
  if (B == 0) return 0;
  if (D > 128 || (D & 1)) return -1;
  if (q_norm == nullptr && k_norm == nullptr) {
    const long long work = (long long)B * (Hq + 2 * Hk) * (D / 2);
    const int grid = (int)((work + 255) / 256);
    return (int)trlb_host::launch_kernel(rope_kv_write_f32_flat_kernel, dim3(grid), dim3(256), 0, st,
                                         trlb_host::pdl_enabled(), acc, row_stride, (const __nv_bfloat16*)bias, seq_lens,
                                         slot_ids, block_table, max_blocks, block_size, (__nv_bfloat16*)q_out,
                                         (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, B, Hq, Hk, D, log2f(theta), v_t, pos_delta);
  }
  const int items = B * (Hq + 2 * Hk);
  const int grid = (items + 7) / 8;
  return (int)trlb_host::launch_kernel(rope_kv_write_f32_kernel, dim3(grid), dim3(256), 0, st, trlb_host::pdl_enabled(), acc,
                                       row_stride, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)q_norm,
                                       (const __nv_bfloat16*)k_norm, norm_eps, seq_lens, slot_ids, block_table, max_blocks,
                                       block_size, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, B, Hq, Hk,
                                       D, log2f(theta), v_t, pos_delta);
}

TRLB_API int trlb_kv_write_prefill(const void* k, const void* v, long long k_stride, long long v_stride,
                                   const int* tok_slot, const int* tok_pos, const int* block_table, int max_blocks,
                                   int block_size, void* kc, void* vc, int T, int Hk, int D, int v_t, cudaStream_t st) {
  if (T == 0) return 0;
  if ((Hk * D) % 8 != 0) return -1;
  const long long work = (long long)T * (Hk * D / 8);
  long long grid = (work + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  kv_write_prefill_kernel<<<(int)grid, 256, 0, st>>>((const __nv_bfloat16*)k, (const __nv_bfloat16*)v, k_stride, v_stride,
                                                     tok_slot, tok_pos, block_table, max_blocks, block_size,
                                                     (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, T, Hk, D, v_t);
  return (int)cudaGetLastError();
}

// scratch sizes: part_o = B*Hq*splits*D floats, part_ml = B*Hq*splits*2 floats
TRLB_API int trlb_paged_decode_attn(const void* q, const void* kc, const void* vc, const int* seq_lens,
                                    const int* slot_ids, const int* block_table, int max_blocks, int block_size, int B,
                                    int Hq, int Hk, int D, float scale, int splits, float* part_o, float* part_ml,
                                    void* out, cudaStream_t st) {
  if (B == 0) return 0;
  if (D != 128 && D != 64) return -1;
  if (Hq % Hk != 0 || Hq / Hk > MAX_G) return -2;
  dim3 grid(B, Hk, splits);
  if (D == 128) {
    paged_decode_attn_kernel<128><<<grid, DEC_THREADS, 0, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)kc,
                                                                (const __nv_bfloat16*)vc, seq_lens, slot_ids, block_table,
                                                                max_blocks, block_size, Hq, Hk, scale, splits, part_o,
                                                                part_ml);
    paged_attn_combine_kernel<128><<<B * Hq, 128, 0, st>>>(part_o, part_ml, splits, (__nv_bfloat16*)out, B * Hq);
  } else {
    return -3;
  }
  return (int)cudaGetLastError();
}

TRLB_API int trlb_sample(const void* logits, int is_bf16, long long row_stride, int B, int V, float inv_temp, float min_p,
                         int eos_id, float eos_floor, unsigned seed, const int* step_ptr, int greedy, int* out_tok,
                         float* out_logp, void* scratch, long long scratch_bytes, cudaStream_t st) {
  if (B == 0) return 0;
  // scratch (optional, zero-initialised once by the caller).  The layout does not depend on B, so calls with
  // different batch sizes never put partials where another call expects its zeroed counters:
  // [4096] row counters | [4096, 8] float4 partials | [4096, 8] int partials
  constexpr long long kRows = 4096, kNeed = kRows * 4 + kRows * 8 * 16 + kRows * 8 * 4;
  if (is_bf16 && min_p <= 0.f && (V % 8) == 0 && (row_stride % 8) == 0 && scratch != nullptr && B <= kRows &&
      scratch_bytes >= kNeed) {
    int S = trlb_host::sm_count() / B;
    S = S < 1 ? 1 : (S > 8 ? 8 : S);
    unsigned* counter = (unsigned*)scratch;
    float4* part = (float4*)((char*)scratch + kRows * 4);
    int* part_i = (int*)(part + kRows * 8);
    sample_split_kernel<<<dim3(B, S), 512, 0, st>>>((const __nv_bfloat16*)logits, row_stride, V, inv_temp, eos_id,
                                                    eos_floor, seed, step_ptr, greedy, part, part_i, counter, out_tok,
                                                    out_logp);
    return (int)cudaGetLastError();
  }
  if (is_bf16)
    sample_kernel<__nv_bfloat16><<<B, 1024, 0, st>>>((const __nv_bfloat16*)logits, row_stride, V, inv_temp, min_p, eos_id,
                                                    eos_floor, seed, step_ptr, greedy, out_tok, out_logp);
  else
    sample_kernel<float><<<B, 1024, 0, st>>>((const float*)logits, row_stride, V, inv_temp, min_p, eos_id, eos_floor,
                                            seed, step_ptr, greedy, out_tok, out_logp);
  return (int)cudaGetLastError();
}

TRLB_API int trlb_advance(const int* tok, const float* logp, const int* slot_ids, int B, int* seq_lens, int* n_gen,
                          int* finished, int* out_tokens, float* out_logps, int max_new, int eos_id, int max_total_len,
                          long long* next_input, int* step_counter, int bump_len, cudaStream_t st) {
  if (B == 0) return 0;
  advance_kernel<<<(B + 127) / 128, 128, 0, st>>>(tok, logp, slot_ids, B, seq_lens, n_gen, finished, out_tokens,
                                                  out_logps, max_new, eos_id, max_total_len, next_input, step_counter, bump_len);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Allocation-free entry point (declared and documented in trlb_no_alloc.h).
//
// For callers that cannot allocate while they launch: a serving loop with a fixed memory budget and
// no allocator, code running where an allocation would synchronise or fail, C programs that link this
// library without PyTorch.  The per-split partials live in the two file-scope arrays below instead of
// in caller-provided buffers.  Every GPU that loads the library carries them (4 MiB + 64 KiB).
// ------------------------------------------------------------------------------------------------
#include <cstdio>

#include "trlb_no_alloc.h"

namespace {
constexpr int kNoAllocD = 128;
static __device__ __align__(256) float g_noalloc_part_o[(size_t)TRLB_NOALLOC_MAX_PARTS * kNoAllocD];
static __device__ __align__(256) float g_noalloc_part_ml[(size_t)TRLB_NOALLOC_MAX_PARTS * 2];

constexpr int kMaxDevices = 64;
// Host-side cache of the arrays' device addresses, one pair per device.  In host code the array names
// above are only stand-ins; the address a kernel may use comes from cudaGetSymbolAddress.
float* g_part_o_addr[kMaxDevices] = {nullptr};
float* g_part_ml_addr[kMaxDevices] = {nullptr};
}  // namespace

TRLB_API int trlb_paged_decode_attn_noalloc(const void* q, const void* kc, const void* vc, const int* seq_lens,
                                            const int* slot_ids, const int* block_table, int max_blocks,
                                            int block_size, int B, int Hq, int Hk, int D, float scale, int splits,
                                            void* out, cudaStream_t st) {
  if (B == 0) return 0;
  if (D != kNoAllocD || Hk <= 0 || Hq % Hk != 0 || Hq / Hk > MAX_G || splits < 1) {
    fprintf(stderr, "trlb_paged_decode_attn_noalloc: unsupported shape (D=%d must be 128, Hq=%d, Hk=%d, splits=%d)\n", D,
            Hq, Hk, splits);
    return TRLB_NOALLOC_ERR_BAD_SHAPE;
  }
  const long long parts = (long long)B * Hq * splits;
  if (parts > TRLB_NOALLOC_MAX_PARTS) {
    fprintf(stderr,
            "trlb_paged_decode_attn_noalloc: B*Hq*splits = %lld exceeds the built-in scratch (%d); use fewer splits, "
            "a smaller batch, or trlb_paged_decode_attn with your own scratch\n",
            parts, TRLB_NOALLOC_MAX_PARTS);
    return TRLB_NOALLOC_ERR_TOO_LARGE;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return TRLB_NOALLOC_ERR_SYMBOL;
  if (g_part_o_addr[dev] == nullptr) {
    // first call on this device: resolve the device addresses (do this before any stream capture)
    float *po = nullptr, *pml = nullptr;
    if (cudaGetSymbolAddress((void**)&po, g_noalloc_part_o) != cudaSuccess ||
        cudaGetSymbolAddress((void**)&pml, g_noalloc_part_ml) != cudaSuccess || po == nullptr || pml == nullptr) {
      fprintf(stderr, "trlb_paged_decode_attn_noalloc: cudaGetSymbolAddress failed on device %d\n", dev);
      return TRLB_NOALLOC_ERR_SYMBOL;
    }
    g_part_ml_addr[dev] = pml;
    g_part_o_addr[dev] = po;
  }
  float* part_o = g_part_o_addr[dev];
  float* part_ml = g_part_ml_addr[dev];
  dim3 grid(B, Hk, splits);
  paged_decode_attn_kernel<128><<<grid, DEC_THREADS, 0, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)kc,
                                                              (const __nv_bfloat16*)vc, seq_lens, slot_ids, block_table,
                                                              max_blocks, block_size, Hq, Hk, scale, splits, part_o,
                                                              part_ml);
  const cudaError_t first = cudaGetLastError();
  if (first != cudaSuccess) return (int)first;  // the combine kernel would read partials that were never written
  paged_attn_combine_kernel<128><<<B * Hq, 128, 0, st>>>(part_o, part_ml, splits, (__nv_bfloat16*)out, B * Hq);
  return (int)cudaGetLastError();
}
