// Memory-bound fused ops: RMSNorm fwd/bwd, RoPE fwd/bwd, SwiGLU fwd/bwd, flat AdamW.
// All are bf16 in / fp32 math, 16-byte vector accesses, sized so a grid covers 148 SMs.
// They replace eager PyTorch / Liger Triton kernels the reference reaches through
// `use_liger_kernel` (trl/trainer/base_config.py:90-95) and torch's fused AdamW.
#include "common.cuh"

namespace trlb {

// ------------------------------------------------------------------------------------------
// RMSNorm forward: y = x * rsqrt(mean(x^2) + eps) * w ; one warp per row, row kept in registers.
// H % 8 == 0, H <= 8192 * 2.
// ------------------------------------------------------------------------------------------
constexpr int RMS_MAX_VEC = 16;  // uint4 per lane => H <= 32 * 16 * 8 = 4096 per pass; larger rows loop twice

template <int VEC_PER_LANE>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                         const __nv_bfloat16* __restrict__ w,
                                                         __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out,
                                                         int T, int H, float eps) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int nvec = H >> 3;
  for (int row = warp; row < T; row += nwarps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
    uint4 buf[VEC_PER_LANE];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VEC_PER_LANE; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        buf[i] = xr[v];
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&buf[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16(u[j]);
          ss += f.x * f.x + f.y * f.y;
        }
      }
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)H + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * H);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
    for (int i = 0; i < VEC_PER_LANE; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        const uint4 wv = wr[v];
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&buf[i]);
        const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wv);
        uint4 o;
        uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = unpack_bf16(u[j]);
          float2 g = unpack_bf16(wu[j]);
          ou[j] = pack_bf16(f.x * rstd * g.x, f.y * rstd * g.y);
        }
        yr[v] = o;
      }
    }
  }
}

// Residual add fused with RMSNorm (inference): res += delta (in place), y = rmsnorm(res) * w.
template <int VEC_PER_LANE>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(__nv_bfloat16* __restrict__ res,
                                                         const __nv_bfloat16* __restrict__ delta,
                                                         const __nv_bfloat16* __restrict__ w,
                                                         __nv_bfloat16* __restrict__ y, int T, int H, float eps) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int nvec = H >> 3;
  for (int row = warp; row < T; row += nwarps) {
    uint4* xr = reinterpret_cast<uint4*>(res + (size_t)row * H);
    const uint4* dr = reinterpret_cast<const uint4*>(delta + (size_t)row * H);
    float buf[VEC_PER_LANE][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VEC_PER_LANE; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        const uint4 a = xr[v], d = dr[v];
        const uint32_t* au = reinterpret_cast<const uint32_t*>(&a);
        const uint32_t* du = reinterpret_cast<const uint32_t*>(&d);
        uint4 o;
        uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16(au[j]), g = unpack_bf16(du[j]);
          ou[j] = pack_bf16(f.x + g.x, f.y + g.y);
          const float2 r = unpack_bf16(ou[j]);  // norm of the value as stored (bf16), like the unfused path
          buf[i][2 * j] = r.x; buf[i][2 * j + 1] = r.y;
          ss += r.x * r.x + r.y * r.y;
        }
        xr[v] = o;
      }
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)H + eps);
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * H);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
    for (int i = 0; i < VEC_PER_LANE; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        const uint4 wv = wr[v];
        const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wv);
        uint4 o;
        uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 g = unpack_bf16(wu[j]);
          ou[j] = pack_bf16(buf[i][2 * j] * rstd * g.x, buf[i][2 * j + 1] * rstd * g.y);
        }
        yr[v] = o;
      }
    }
  }
}

// Same op for few rows (decode batches): one CTA per row, so 64 rows still occupy 64 SMs with 8
// warps each instead of 8 CTAs.  delta may be null (plain RMSNorm).  H <= 256 * 8 * VPT.
template <int VPT>
__global__ void __launch_bounds__(256) add_rmsnorm_row_kernel(__nv_bfloat16* __restrict__ res,
                                                             const __nv_bfloat16* __restrict__ delta,
                                                             const __nv_bfloat16* __restrict__ w,
                                                             __nv_bfloat16* __restrict__ y, int H, float eps) {
  __shared__ float red[8];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int nvec = H >> 3;
  uint4* xr = reinterpret_cast<uint4*>(res + (size_t)row * H);
  float buf[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * 256;
    if (v < nvec) {
      uint4 a = xr[v];
      uint32_t* au = reinterpret_cast<uint32_t*>(&a);
      if (delta != nullptr) {
        const uint4 d = reinterpret_cast<const uint4*>(delta + (size_t)row * H)[v];
        const uint32_t* du = reinterpret_cast<const uint32_t*>(&d);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16(au[j]), g = unpack_bf16(du[j]);
          au[j] = pack_bf16(f.x + g.x, f.y + g.y);
        }
        xr[v] = a;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 r = unpack_bf16(au[j]);
        buf[i][2 * j] = r.x; buf[i][2 * j + 1] = r.y;
        ss += r.x * r.x + r.y * r.y;
      }
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) red[wid] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) tot += red[k];
  const float rstd = rsqrtf(tot / (float)H + eps);
  uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * H);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * 256;
    if (v < nvec) {
      const uint4 wv = wr[v];
      const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wv);
      uint4 o;
      uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 g = unpack_bf16(wu[j]);
        ou[j] = pack_bf16(buf[i][2 * j] * rstd * g.x, buf[i][2 * j + 1] * rstd * g.y);
      }
      yr[v] = o;
    }
  }
}

// Variant for the split-K decode GEMM: delta holds fp32 sums; they are consumed (added to the residual stream) and
// cleared here, so the next GEMM that accumulates into the same buffer starts from zero without a memset launch.
template <int VPT>
__global__ void __launch_bounds__(256) add_rmsnorm_f32_row_kernel(__nv_bfloat16* __restrict__ res,
                                                                 float* __restrict__ delta,
                                                                 const __nv_bfloat16* __restrict__ w,
                                                                 __nv_bfloat16* __restrict__ y, int H, float eps) {
  __shared__ float red[8];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int nvec = H >> 3;
  uint4* xr = reinterpret_cast<uint4*>(res + (size_t)row * H);
  float4* dr = reinterpret_cast<float4*>(delta + (size_t)row * H);
  float buf[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * 256;
    if (v < nvec) {
      uint4 a = xr[v];
      uint32_t* au = reinterpret_cast<uint32_t*>(&a);
      const float4 d0 = dr[2 * v], d1 = dr[2 * v + 1];
      dr[2 * v] = make_float4(0.f, 0.f, 0.f, 0.f);
      dr[2 * v + 1] = make_float4(0.f, 0.f, 0.f, 0.f);
      const float dv[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16(au[j]);
        au[j] = pack_bf16(f.x + dv[2 * j], f.y + dv[2 * j + 1]);
      }
      xr[v] = a;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 r = unpack_bf16(au[j]);
        buf[i][2 * j] = r.x; buf[i][2 * j + 1] = r.y;
        ss += r.x * r.x + r.y * r.y;
      }
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) red[wid] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) tot += red[k];
  const float rstd = rsqrtf(tot / (float)H + eps);
  uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * H);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * 256;
    if (v < nvec) {
      const uint4 wv = wr[v];
      const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wv);
      uint4 o;
      uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 g = unpack_bf16(wu[j]);
        ou[j] = pack_bf16(buf[i][2 * j] * rstd * g.x, buf[i][2 * j + 1] * rstd * g.y);
      }
      yr[v] = o;
    }
  }
}

// RMSNorm backward.  dx = rstd * (w*dy - x * rstd^2 * mean(w*dy*x)).  A CTA walks its rows one at a
// time; thread t owns the same columns for every row, so the dw partial sums stay in registers.
// Per-CTA partials go to fp32 scratch [gridDim.x, H], reduced by rmsnorm_dw_reduce_kernel.
template <int VPT>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                         const __nv_bfloat16* __restrict__ x,
                                                         const __nv_bfloat16* __restrict__ w,
                                                         const float* __restrict__ rstd_in,
                                                         __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_part,
                                                         int T, int H) {
  __shared__ float red[2][8];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int nvec = H >> 3;
  float dwacc[VPT][8], wv[VPT][8];
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * 256;
    uint4 c = make_uint4(0, 0, 0, 0);
    if (v < nvec) c = wr[v];
    const uint32_t* cu = reinterpret_cast<const uint32_t*>(&c);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf16(cu[j]);
      wv[i][2 * j] = f.x; wv[i][2 * j + 1] = f.y;
      dwacc[i][2 * j] = 0.f; dwacc[i][2 * j + 1] = 0.f;
    }
  }
  int it = 0;
  for (int row = blockIdx.x; row < T; row += gridDim.x, ++it) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + (size_t)row * H);
    const float rstd = rstd_in[row];
    float xv[VPT][8], gv[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = tid + i * 256;
      uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0, 0, 0);
      if (v < nvec) { a = xr[v]; b = gr[v]; }
      const uint32_t* au = reinterpret_cast<const uint32_t*>(&a);
      const uint32_t* bu = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fx = unpack_bf16(au[j]), fg = unpack_bf16(bu[j]);
        xv[i][2 * j] = fx.x; xv[i][2 * j + 1] = fx.y;
        dwacc[i][2 * j] += fg.x * fx.x * rstd;
        dwacc[i][2 * j + 1] += fg.y * fx.y * rstd;
        gv[i][2 * j] = fg.x * wv[i][2 * j]; gv[i][2 * j + 1] = fg.y * wv[i][2 * j + 1];
        dot += gv[i][2 * j] * fx.x + gv[i][2 * j + 1] * fx.y;
      }
    }
    dot = warp_sum(dot);
    float* rbuf = red[it & 1];  // double-buffered: one barrier per row is enough
    if (lane == 0) rbuf[wid] = dot;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) tot += rbuf[k];
    const float coef = tot * rstd * rstd / (float)H;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * H);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = tid + i * 256;
      if (v < nvec) {
        uint4 o;
        uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          ou[j] = pack_bf16(rstd * (gv[i][2 * j] - xv[i][2 * j] * coef),
                            rstd * (gv[i][2 * j + 1] - xv[i][2 * j + 1] * coef));
        dxr[v] = o;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = tid + i * 256;
    if (v < nvec) {
      float4* dst = reinterpret_cast<float4*>(dw_part + (size_t)blockIdx.x * H + (size_t)v * 8);
      dst[0] = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      dst[1] = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
}

__global__ void rmsnorm_dw_reduce_kernel(const float* __restrict__ part, int nparts, int H, float* __restrict__ dw_f32,
                                         __nv_bfloat16* __restrict__ dw_bf16) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= H) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += part[(size_t)p * H + i];
  if (dw_f32) dw_f32[i] = s;
  if (dw_bf16) dw_bf16[i] = __float2bfloat16(s);
}

// ------------------------------------------------------------------------------------------
// RoPE (rotate-half) on q [T,Hq,D] and k [T,Hk,D] read through a row stride (views of the fused
// QKV output) and written densely.  sign = +1 forward, -1 backward (inverse rotation).
// ------------------------------------------------------------------------------------------
template <bool MULTI>
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                            long long q_row_stride, long long k_row_stride, const int* __restrict__ pos,
                            __nv_bfloat16* __restrict__ qo, __nv_bfloat16* __restrict__ ko, int T, int Hq, int Hk, int D,
                            float log2_theta, float sign, const int* __restrict__ row_of_freq) {
  const int half = D >> 1;
  const int pairs_per_tok = (Hq + Hk) * (half >> 1);  // two frequencies per thread
  const long long total = (long long)T * pairs_per_tok;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / pairs_per_tok);
    int r = (int)(idx % pairs_per_tok);
    const int head = r / (half >> 1);
    const int f = (r % (half >> 1)) * 2;
    // MULTI: pos is [rows, T] and frequency f turns with the position row row_of_freq[f] (multimodal RoPE)
    const float p0 = MULTI ? (float)pos[(size_t)row_of_freq[f] * T + t] : (float)pos[t];
    const float p1 = MULTI ? (float)pos[(size_t)row_of_freq[f + 1] * T + t] : p0;
    const float inv0 = exp2f(-log2_theta * (float)(2 * f) / (float)D);
    const float inv1 = exp2f(-log2_theta * (float)(2 * f + 2) / (float)D);
    float s0, c0, s1, c1;
    sincosf(p0 * inv0, &s0, &c0);
    sincosf(p1 * inv1, &s1, &c1);
    s0 *= sign; s1 *= sign;
    const __nv_bfloat16* src;
    __nv_bfloat16* dst;
    if (head < Hq) {
      src = q + (size_t)t * q_row_stride + (size_t)head * D;
      dst = qo + ((size_t)t * Hq + head) * D;
    } else {
      src = k + (size_t)t * k_row_stride + (size_t)(head - Hq) * D;
      dst = ko + ((size_t)t * Hk + (head - Hq)) * D;
    }
    const float2 lo = unpack_bf16(*reinterpret_cast<const uint32_t*>(src + f));
    const float2 hi = unpack_bf16(*reinterpret_cast<const uint32_t*>(src + half + f));
    *reinterpret_cast<uint32_t*>(dst + f) = pack_bf16(lo.x * c0 - hi.x * s0, lo.y * c1 - hi.y * s1);
    *reinterpret_cast<uint32_t*>(dst + half + f) = pack_bf16(hi.x * c0 + lo.x * s0, hi.y * c1 + lo.y * s1);
  }
}

// ------------------------------------------------------------------------------------------
// SwiGLU: out[t, i] = silu(gu[t, i]) * gu[t, I + i]
// ------------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long long T,
                                  int I) {
  const int nvec = I >> 3;
  const long long total = T * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int v = (int)(idx % nvec);
    const uint4 g = reinterpret_cast<const uint4*>(gu + t * 2 * I)[v];
    const uint4 u = reinterpret_cast<const uint4*>(gu + t * 2 * I + I)[v];
    const uint32_t* gp = reinterpret_cast<const uint32_t*>(&g);
    const uint32_t* up = reinterpret_cast<const uint32_t*>(&u);
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16(gp[j]), b = unpack_bf16(up[j]);
      op[j] = pack_bf16(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y);
    }
    reinterpret_cast<uint4*>(out + t * I)[v] = o;
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int I) {
  const int nvec = I >> 3;
  const long long total = T * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int v = (int)(idx % nvec);
    const uint4 g = reinterpret_cast<const uint4*>(gu + t * 2 * I)[v];
    const uint4 u = reinterpret_cast<const uint4*>(gu + t * 2 * I + I)[v];
    const uint4 d = reinterpret_cast<const uint4*>(dout + t * I)[v];
    const uint32_t* gp = reinterpret_cast<const uint32_t*>(&g);
    const uint32_t* up = reinterpret_cast<const uint32_t*>(&u);
    const uint32_t* dp = reinterpret_cast<const uint32_t*>(&d);
    uint4 og, ou;
    uint32_t* ogp = reinterpret_cast<uint32_t*>(&og);
    uint32_t* oup = reinterpret_cast<uint32_t*>(&ou);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16(gp[j]), b = unpack_bf16(up[j]), dd = unpack_bf16(dp[j]);
      const float s0 = 1.f / (1.f + __expf(-a.x)), s1 = 1.f / (1.f + __expf(-a.y));
      const float silu0 = a.x * s0, silu1 = a.y * s1;
      ogp[j] = pack_bf16(dd.x * b.x * (s0 + silu0 * (1.f - s0)), dd.y * b.y * (s1 + silu1 * (1.f - s1)));
      oup[j] = pack_bf16(dd.x * silu0, dd.y * silu1);
    }
    reinterpret_cast<uint4*>(dgu + t * 2 * I)[v] = og;
    reinterpret_cast<uint4*>(dgu + t * 2 * I + I)[v] = ou;
  }
}

// ------------------------------------------------------------------------------------------
// Flat AdamW on an fp32 master shard; refreshes the bf16 compute copy in the same pass.
// grad may be fp32 or bf16.  grad_scale is read from device memory when a pointer is given
// (clip coefficient computed on the device: no host sync between norm and update).
// ------------------------------------------------------------------------------------------
template <typename GradT>
__global__ void adamw_kernel(float* __restrict__ master, const GradT* __restrict__ grad, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ shadow, long long n, float lr, float b1,
                             float b2, float eps, float wd, float bc1, float bc2_sqrt, float grad_scale,
                             const float* __restrict__ grad_scale_ptr) {
  const float gs = grad_scale_ptr ? grad_scale * (*grad_scale_ptr) : grad_scale;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float g;
    if constexpr (sizeof(GradT) == 2) g = __bfloat162float(grad[i]) * gs; else g = (float)grad[i] * gs;
    float mi = m[i] * b1 + (1.f - b1) * g;
    float vi = v[i] * b2 + (1.f - b2) * g * g;
    m[i] = mi;
    v[i] = vi;
    float p = master[i];
    p -= lr * wd * p;
    p -= (lr / bc1) * mi / (sqrtf(vi) / bc2_sqrt + eps);
    master[i] = p;
    if (shadow) shadow[i] = __float2bfloat16(p);
  }
}

// Same update, four elements per thread and iteration through 16-byte loads / stores (8 bytes for bf16 operands):
// the scalar kernel keeps only four 4-byte loads in flight per thread and reached 0.69 of the copy bandwidth; the
// host picks this one when every pointer is 16-byte aligned (the tail of n % 4 elements goes to the scalar kernel).
template <typename GradT>
__global__ void __launch_bounds__(256)
adamw_vec4_kernel(float* __restrict__ master, const GradT* __restrict__ grad, float* __restrict__ m,
                  float* __restrict__ v, __nv_bfloat16* __restrict__ shadow, long long n4, float lr, float b1, float b2,
                  float eps, float wd, float bc1, float bc2_sqrt, float grad_scale,
                  const float* __restrict__ grad_scale_ptr) {
  const float gs = grad_scale_ptr ? grad_scale * (*grad_scale_ptr) : grad_scale;
  const float step = lr / bc1, decay = 1.f - lr * wd;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float g[4];
    if constexpr (sizeof(GradT) == 2) {
      const uint2 raw = reinterpret_cast<const uint2*>(grad)[i];
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
      const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
      g[0] = __low2float(lo); g[1] = __high2float(lo); g[2] = __low2float(hi); g[3] = __high2float(hi);
    } else {
      const float4 r = reinterpret_cast<const float4*>(grad)[i];
      g[0] = r.x; g[1] = r.y; g[2] = r.z; g[3] = r.w;
    }
    float4 m4 = reinterpret_cast<const float4*>(m)[i];
    float4 v4 = reinterpret_cast<const float4*>(v)[i];
    float4 p4 = reinterpret_cast<const float4*>(master)[i];
    float* mm = reinterpret_cast<float*>(&m4);
    float* vv = reinterpret_cast<float*>(&v4);
    float* pp = reinterpret_cast<float*>(&p4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = g[j] * gs;
      mm[j] = mm[j] * b1 + (1.f - b1) * gj;
      vv[j] = vv[j] * b2 + (1.f - b2) * gj * gj;
      float pj = pp[j] * decay;
      pj -= step * mm[j] / (sqrtf(vv[j]) / bc2_sqrt + eps);
      pp[j] = pj;
    }
    reinterpret_cast<float4*>(m)[i] = m4;
    reinterpret_cast<float4*>(v)[i] = v4;
    reinterpret_cast<float4*>(master)[i] = p4;
    if (shadow) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(pp[0], pp[1]), hi = __floats2bfloat162_rn(pp[2], pp[3]);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(shadow)[i] = o;
    }
  }
}

// sum of squares of a flat gradient buffer -> out[0] (atomic accumulate; zero it first)
template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ x, long long n, float* __restrict__ out) {
  float s = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float f;
    if constexpr (sizeof(T) == 2) f = __bfloat162float(x[i]); else f = (float)x[i];
    s += f * f;
  }
  s = warp_sum(s);
  __shared__ float ws[32];
  if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? ws[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) atomicAdd(out, s);
  }
}

}  // namespace trlb

using namespace trlb;

static inline int grid_for(long long work, int threads, int per_sm = 8) {
  long long g = (work + threads - 1) / threads;
  long long cap = (long long)trlb_host::sm_count() * per_sm;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

TRLB_API int trlb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int T, int H, float eps,
                              cudaStream_t st) {
  if (T == 0) return 0;
  if (H % 8 != 0 || H > 32 * 8 * RMS_MAX_VEC * 2) return -1;
  const int threads = 256;
  const int grid = grid_for((long long)T * 32, threads);
  const int vec = (H / 8 + 31) / 32;
  auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w; auto Y = (__nv_bfloat16*)y;
  if (vec <= 1) rmsnorm_fwd_kernel<1><<<grid, threads, 0, st>>>(X, W, Y, rstd, T, H, eps);
  else if (vec <= 2) rmsnorm_fwd_kernel<2><<<grid, threads, 0, st>>>(X, W, Y, rstd, T, H, eps);
  else if (vec <= 4) rmsnorm_fwd_kernel<4><<<grid, threads, 0, st>>>(X, W, Y, rstd, T, H, eps);
  else if (vec <= 8) rmsnorm_fwd_kernel<8><<<grid, threads, 0, st>>>(X, W, Y, rstd, T, H, eps);
  else if (vec <= 16) rmsnorm_fwd_kernel<16><<<grid, threads, 0, st>>>(X, W, Y, rstd, T, H, eps);
  else rmsnorm_fwd_kernel<32><<<grid, threads, 0, st>>>(X, W, Y, rstd, T, H, eps);
  return (int)cudaGetLastError();
}

// main-gradient accumulation: dst (fp32) += src (bf16), 8 elements per thread iteration
__global__ void __launch_bounds__(256) accum_bf16_f32_kernel(float* __restrict__ dst, const __nv_bfloat16* __restrict__ src,
                                                            long long n) {
  const long long nvec = n >> 3;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec; v += stride) {
    const uint4 s = reinterpret_cast<const uint4*>(src)[v];
    const uint32_t su[4] = {s.x, s.y, s.z, s.w};
    float4 a = reinterpret_cast<float4*>(dst)[2 * v], b = reinterpret_cast<float4*>(dst)[2 * v + 1];
    const float2 f0 = unpack_bf16(su[0]), f1 = unpack_bf16(su[1]), f2 = unpack_bf16(su[2]), f3 = unpack_bf16(su[3]);
    a.x += f0.x; a.y += f0.y; a.z += f1.x; a.w += f1.y;
    b.x += f2.x; b.y += f2.y; b.z += f3.x; b.w += f3.y;
    reinterpret_cast<float4*>(dst)[2 * v] = a;
    reinterpret_cast<float4*>(dst)[2 * v + 1] = b;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
    const long long i = (nvec << 3) + threadIdx.x;
    dst[i] += __bfloat162float(src[i]);
  }
}

TRLB_API int trlb_accum_bf16_f32(float* dst, const void* src, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(dst) & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) return -2;
  long long blocks = ((n >> 3) + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 16) blocks = 148 * 16;
  accum_bf16_f32_kernel<<<(int)blocks, 256, 0, st>>>(dst, (const __nv_bfloat16*)src, n);
  return (int)cudaGetLastError();
}

// res[T,H] += delta32[T,H] (fp32 sums, cleared afterwards), y = rmsnorm(res) * w  (H <= 8192, few rows)
TRLB_API int trlb_add_rmsnorm_f32(void* res, float* delta, const void* w, void* y, int T, int H, float eps,
                                  cudaStream_t st) {
  if (T == 0) return 0;
  if (H % 8 != 0 || H > 8192) return -1;
  auto R = (__nv_bfloat16*)res; auto W = (const __nv_bfloat16*)w; auto Y = (__nv_bfloat16*)y;
  const int vpt = (H / 8 + 255) / 256;
  const bool pdl = trlb_host::pdl_enabled();
  auto kern = vpt <= 1 ? add_rmsnorm_f32_row_kernel<1> : (vpt <= 2 ? add_rmsnorm_f32_row_kernel<2> : add_rmsnorm_f32_row_kernel<4>);
  return (int)trlb_host::launch_kernel(kern, dim3(T), dim3(256), 0, st, pdl, R, delta, W, Y, H, eps);
}

// res[T,H] += delta[T,H] in place, y = rmsnorm(res) * w  (H <= 8192)
TRLB_API int trlb_add_rmsnorm(void* res, const void* delta, const void* w, void* y, int T, int H, float eps,
                              cudaStream_t st) {
  if (T == 0) return 0;
  if (H % 8 != 0 || H > 8192) return -1;
  if (T <= 4 * trlb_host::sm_count() || H > 4096) {
    auto R = (__nv_bfloat16*)res; auto Dl = (const __nv_bfloat16*)delta; auto W = (const __nv_bfloat16*)w;
    auto Y = (__nv_bfloat16*)y;
    const int vpt = (H / 8 + 255) / 256;
    if (vpt <= 1) add_rmsnorm_row_kernel<1><<<T, 256, 0, st>>>(R, Dl, W, Y, H, eps);
    else if (vpt <= 2) add_rmsnorm_row_kernel<2><<<T, 256, 0, st>>>(R, Dl, W, Y, H, eps);
    else add_rmsnorm_row_kernel<4><<<T, 256, 0, st>>>(R, Dl, W, Y, H, eps);
    return (int)cudaGetLastError();
  }
  const int threads = 256;
  const int grid = grid_for((long long)T * 32, threads);
  const int vec = (H / 8 + 31) / 32;
  auto R = (__nv_bfloat16*)res; auto Dl = (const __nv_bfloat16*)delta; auto W = (const __nv_bfloat16*)w;
  auto Y = (__nv_bfloat16*)y;
  if (vec <= 2) add_rmsnorm_kernel<2><<<grid, threads, 0, st>>>(R, Dl, W, Y, T, H, eps);
  else if (vec <= 4) add_rmsnorm_kernel<4><<<grid, threads, 0, st>>>(R, Dl, W, Y, T, H, eps);
  else if (vec <= 8) add_rmsnorm_kernel<8><<<grid, threads, 0, st>>>(R, Dl, W, Y, T, H, eps);
  else add_rmsnorm_kernel<16><<<grid, threads, 0, st>>>(R, Dl, W, Y, T, H, eps);
  return (int)cudaGetLastError();
}

// Number of partial rows the backward writes into dw_part (caller sizes scratch = parts * H floats).
TRLB_API int trlb_rmsnorm_bwd_parts(int T) {
  int cap = trlb_host::sm_count() * 4;
  return T < 1 ? 1 : (T > cap ? cap : T);
}

TRLB_API int trlb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw_part,
                              float* dw_f32, void* dw_bf16, int T, int H, cudaStream_t st) {
  if (T == 0) return 0;
  if (H % 8 != 0 || H > 8192) return -1;
  const int grid = trlb_rmsnorm_bwd_parts(T);
  const int vpt = (H / 8 + 255) / 256;
  auto DY = (const __nv_bfloat16*)dy; auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w;
  auto DX = (__nv_bfloat16*)dx;
  if (vpt <= 1) rmsnorm_bwd_kernel<1><<<grid, 256, 0, st>>>(DY, X, W, rstd, DX, dw_part, T, H);
  else if (vpt <= 2) rmsnorm_bwd_kernel<2><<<grid, 256, 0, st>>>(DY, X, W, rstd, DX, dw_part, T, H);
  else rmsnorm_bwd_kernel<4><<<grid, 256, 0, st>>>(DY, X, W, rstd, DX, dw_part, T, H);
  rmsnorm_dw_reduce_kernel<<<(H + 255) / 256, 256, 0, st>>>(dw_part, grid, H, dw_f32, (__nv_bfloat16*)dw_bf16);
  return (int)cudaGetLastError();
}

TRLB_API int trlb_rope(const void* q, const void* k, long long q_row_stride, long long k_row_stride, const int* pos,
                       void* qo, void* ko, int T, int Hq, int Hk, int D, float theta, float sign, cudaStream_t st) {
  if (T == 0) return 0;
  if (D % 4 != 0) return -1;
  const long long work = (long long)T * (Hq + Hk) * (D / 4);
  rope_kernel<false><<<grid_for(work, 256), 256, 0, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, q_row_stride,
                                                          k_row_stride, pos, (__nv_bfloat16*)qo, (__nv_bfloat16*)ko, T, Hq,
                                                          Hk, D, log2f(theta), sign, nullptr);
  return (int)cudaGetLastError();
}

// Multimodal RoPE: pos3 [rows, T] int32 (temporal / height / width positions), row_of_freq [D / 2] int32 says which
// row turns each rotary frequency.
TRLB_API int trlb_rope_multi(const void* q, const void* k, long long q_row_stride, long long k_row_stride, const int* pos3,
                             const int* row_of_freq, void* qo, void* ko, int T, int Hq, int Hk, int D, float theta,
                             float sign, cudaStream_t st) {
  if (T == 0) return 0;
  if (D % 4 != 0) return -1;
  const long long work = (long long)T * (Hq + Hk) * (D / 4);
  rope_kernel<true><<<grid_for(work, 256), 256, 0, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, q_row_stride,
                                                         k_row_stride, pos3, (__nv_bfloat16*)qo, (__nv_bfloat16*)ko, T, Hq,
                                                         Hk, D, log2f(theta), sign, row_of_freq);
  return (int)cudaGetLastError();
}

TRLB_API int trlb_swiglu_fwd(const void* gu, void* out, long long T, int I, cudaStream_t st) {
  if (T == 0) return 0;
  if (I % 8 != 0) return -1;
  swiglu_fwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, st>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, I);
  return (int)cudaGetLastError();
}

TRLB_API int trlb_swiglu_bwd(const void* dout, const void* gu, void* dgu, long long T, int I, cudaStream_t st) {
  if (T == 0) return 0;
  if (I % 8 != 0) return -1;
  swiglu_bwd_kernel<<<grid_for(T * (I / 8), 256), 256, 0, st>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)gu,
                                                               (__nv_bfloat16*)dgu, T, I);
  return (int)cudaGetLastError();
}

TRLB_API int trlb_adamw(float* master, const void* grad, int grad_is_bf16, float* m, float* v, void* shadow, long long n,
                        int step, float lr, float b1, float b2, float eps, float wd, float grad_scale,
                        const float* grad_scale_ptr, cudaStream_t st) {
  if (n == 0) return 0;
  const float bc1 = 1.f - powf(b1, (float)step);
  const float bc2s = sqrtf(1.f - powf(b2, (float)step));
  const auto misaligned = [](const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; };
  const bool vec = n >= 4 && !misaligned(master, 16) && !misaligned(m, 16) && !misaligned(v, 16) &&
                   !misaligned(grad, grad_is_bf16 ? 8 : 16) && (!shadow || !misaligned(shadow, 8));
  const long long n4 = vec ? n / 4 : 0, done = n4 * 4;
  if (n4 > 0) {
    const int grid = grid_for(n4, 256, 8);
    if (grad_is_bf16)
      adamw_vec4_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(master, (const __nv_bfloat16*)grad, m, v,
                                                            (__nv_bfloat16*)shadow, n4, lr, b1, b2, eps, wd, bc1, bc2s,
                                                            grad_scale, grad_scale_ptr);
    else
      adamw_vec4_kernel<float><<<grid, 256, 0, st>>>(master, (const float*)grad, m, v, (__nv_bfloat16*)shadow, n4, lr, b1,
                                                    b2, eps, wd, bc1, bc2s, grad_scale, grad_scale_ptr);
  }
  if (done < n) {  // unaligned buffers, or the last n % 4 elements
    const long long r = n - done;
    const int grid = grid_for(r, 256, 16);
    __nv_bfloat16* sh = shadow ? (__nv_bfloat16*)shadow + done : nullptr;
    if (grad_is_bf16)
      adamw_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(master + done, (const __nv_bfloat16*)grad + done, m + done,
                                                       v + done, sh, r, lr, b1, b2, eps, wd, bc1, bc2s, grad_scale,
                                                       grad_scale_ptr);
    else
      adamw_kernel<float><<<grid, 256, 0, st>>>(master + done, (const float*)grad + done, m + done, v + done, sh, r, lr,
                                                b1, b2, eps, wd, bc1, bc2s, grad_scale, grad_scale_ptr);
  }
  return (int)cudaGetLastError();
}

TRLB_API int trlb_sumsq(const void* x, int is_bf16, long long n, float* out, cudaStream_t st) {
  if (n == 0) return 0;
  const int grid = grid_for(n, 256, 8);
  if (is_bf16) sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, n, out);
  else sumsq_kernel<float><<<grid, 256, 0, st>>>((const float*)x, n, out);
  return (int)cudaGetLastError();
}
