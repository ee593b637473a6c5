// Collectives fused with their compute, over NVLink peer memory (symmetric buffers mapped by every
// rank of the node).  Peer data is reached with plain ld/st on peer pointers or with multimem.*
// (NVSwitch reduce / broadcast) on the multicast mapping of the same buffers.  There is no TMA in
// this file.
//
//   rs_reduce        gradient reduce-scatter fused with the fp32 cast, the 1/world scale and the
//                    squared-norm partial of this rank's shard
//   adamw_bcast      sharded AdamW on the reduced shard, writing the updated bf16 parameters straight
//                    into every rank's replica (the parameter all-gather happens in the store)
//   shard_allgather  parameter all-gather by pull (peer loads) or push (multimem.st)
//   shard_pull       a layer's parameter slices pulled from every owner into a local full-size slot (streamed
//                    full shard: no barrier, the slices only change at the optimizer step)
//   allreduce_add_rmsnorm   TP decode: sum of the ranks' partial GEMM outputs + residual add + RMSNorm
//   norm_allreduce   grad-norm partials of all ranks -> clip coefficient on every rank, no host sync
//
// Cross-GPU ordering uses a signal pad (one 32-bit word per (channel, peer)) written with
// st.release.sys and polled with ld.acquire.sys.  Every poll is bounded by time: when it runs out the
// kernel records ERR_WAIT_TIMEOUT in the status words and returns, the context stays usable.
//
// They replace NCCL reduce-scatter + torch fused AdamW + NCCL all-gather of the reference's
// DeepSpeed/FSDP engines (trl/models/utils.py:236-321, trl/accelerate_configs/zero*.yaml) and the
// per-layer all-reduce inside vLLM's tensor-parallel decode (trl/generation/vllm_generation.py:324-332).
#include "common.cuh"

namespace trlb {

constexpr int MAX_PEERS = 8;
struct Peers {
  void* buf[MAX_PEERS];       // the same symmetric buffer on every rank
  uint32_t* pad[MAX_PEERS];   // signal pads
  int rank, world;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

constexpr uint64_t kPeerWaitNs = 1000ull * 1000ull * 1000ull;  // 1 s: a peer that is this late is gone

// All ranks meet: block 0 announces `epoch` on `channel` to every peer and waits for theirs, then
// releases the other blocks of this grid through `local_gate`.  The grid must be co-resident
// (launchers cap it at the SM count).  Returns false if a wait timed out.
__device__ bool peers_barrier(const Peers& P, int channel, uint32_t epoch, uint32_t* local_gate, int* status, int site) {
  __shared__ int ok_s;
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) ok_s = 1;
    __syncthreads();
    if (threadIdx.x < P.world) {
      __threadfence_system();
      st_release_sys(P.pad[threadIdx.x] + channel * MAX_PEERS + P.rank, epoch);
      const uint32_t* mine = P.pad[P.rank] + channel * MAX_PEERS + threadIdx.x;
      const uint64_t t0 = globaltimer_ns();
      while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
        if (globaltimer_ns() - t0 > kPeerWaitNs) {
          report_error(status, ERR_WAIT_TIMEOUT, site, (int)threadIdx.x);
          ok_s = 0;
          break;
        }
        __nanosleep(64);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      atomicExch(local_gate, ok_s ? epoch : 0xFFFFFFFFu);
    }
    return ok_s != 0;
  }
  if (threadIdx.x == 0) {
    ok_s = 1;
    const uint64_t t0 = globaltimer_ns();
    while (true) {
      const uint32_t g = ld_acquire_gpu(local_gate);
      if (g == 0xFFFFFFFFu) { ok_s = 0; break; }
      if ((int32_t)(g - epoch) >= 0) break;
      if (globaltimer_ns() - t0 > 2 * kPeerWaitNs) {
        report_error(status, ERR_WAIT_TIMEOUT, site + 1, (int)blockIdx.x);
        ok_s = 0;
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return ok_s != 0;
}

// True in exactly one block of the grid: the last one to get here.  Used to publish the new epoch only
// after every block has read the old one (a block that starts late must not see the bumped counter).
__device__ bool grid_last_block(uint32_t* counter) {
  __shared__ unsigned last_s;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last_s = atomicAdd(counter, 1u);
  __syncthreads();
  if (last_s == gridDim.x - 1) {
    if (threadIdx.x == 0) *counter = 0;
    return true;
  }
  return false;
}

// ------------------------------------------------------------------------------------------------
// rs_reduce: out[i] = (1/world) * sum_p grad_p[lo + i]  (fp32), sumsq += out[i]^2.
// grad buffers are fp32 (GradT=float) or bf16.  When `mc` is given (multicast mapping of the gradient
// buffer) the sum is done by the switch: multimem.ld_reduce.
// ------------------------------------------------------------------------------------------------
template <typename GradT>
__global__ void __launch_bounds__(512)
rs_reduce_kernel(Peers P, const void* mc, long long lo, long long n, float* __restrict__ out, float* __restrict__ sumsq,
                 uint32_t* epoch_ctr, uint32_t* local_gate, int channel, int* status, int accumulate) {
  const uint32_t epoch = *epoch_ctr + 1;
  if (!peers_barrier(P, channel, epoch, local_gate, status, 500)) return;
  const float inv = 1.f / (float)P.world;
  float ss = 0.f;
  constexpr int VEC = 16 / sizeof(GradT);  // elements per 16-byte access
  const long long nvec = n / VEC;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
    if (mc != nullptr && sizeof(GradT) == 4) {
      const float* src = reinterpret_cast<const float*>(mc) + lo + v * VEC;
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(acc[0]), "=f"(acc[1]), "=f"(acc[2]), "=f"(acc[3])
                   : "l"(src)
                   : "memory");
    } else {
      uint4 raw[MAX_PEERS];
#pragma unroll
      for (int p = 0; p < MAX_PEERS; ++p)
        if (p < P.world) raw[p] = reinterpret_cast<const uint4*>(reinterpret_cast<const GradT*>(P.buf[p]) + lo)[v];
#pragma unroll
      for (int p = 0; p < MAX_PEERS; ++p) {
        if (p < P.world) {
          if constexpr (sizeof(GradT) == 4) {
            const float* f = reinterpret_cast<const float*>(&raw[p]);
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] += f[j];
          } else {
            const uint32_t* u = reinterpret_cast<const uint32_t*>(&raw[p]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = unpack_bf16(u[j]);
              acc[2 * j] += f.x;
              acc[2 * j + 1] += f.y;
            }
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      acc[j] *= inv;
      ss += acc[j] * acc[j];
    }
    float4* dst = reinterpret_cast<float4*>(out + v * VEC);
    if (accumulate) {  // out += mean (the accumulator of several micro-batches)
      const float4 o0 = dst[0];
      acc[0] += o0.x; acc[1] += o0.y; acc[2] += o0.z; acc[3] += o0.w;
      if constexpr (VEC == 8) {
        const float4 o1 = dst[1];
        acc[4] += o1.x; acc[5] += o1.y; acc[6] += o1.z; acc[7] += o1.w;
      }
    }
    dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    if constexpr (VEC == 8) dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  ss = warp_sum(ss);
  __shared__ float ws[16];
  if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += ws[w];
    atomicAdd(sumsq, t);
  }
  if (grid_last_block(local_gate + 1) && threadIdx.x == 0) *epoch_ctr = epoch;
}

// ------------------------------------------------------------------------------------------------
// norm_allreduce: every rank publishes its sum of squares into slot [rank] of every peer's `slots`
// (symmetric, world floats), then computes norm and clip coefficient locally.  One CTA.
// ------------------------------------------------------------------------------------------------
__global__ void norm_allreduce_kernel(Peers P, const float* __restrict__ my_sumsq, float max_norm,
                                      float* __restrict__ norm_out, float* __restrict__ clip_out, uint32_t* epoch_ctr,
                                      uint32_t* local_gate, int channel, int* status) {
  const uint32_t epoch = *epoch_ctr + 1;
  if (threadIdx.x < P.world) reinterpret_cast<float*>(P.buf[threadIdx.x])[P.rank] = *my_sumsq;
  __syncthreads();
  if (!peers_barrier(P, channel, epoch, local_gate, status, 520)) return;
  if (threadIdx.x == 0) {
    float t = 0.f;
    const float* mine = reinterpret_cast<const float*>(P.buf[P.rank]);
    for (int p = 0; p < P.world; ++p) t += mine[p];
    const float nrm = sqrtf(t);
    *norm_out = nrm;
    *clip_out = (max_norm > 0.f) ? fminf(1.f, max_norm / (nrm + 1e-6f)) : 1.f;
    *epoch_ctr = epoch;
  }
}

// ------------------------------------------------------------------------------------------------
// adamw_bcast: AdamW on this rank's shard; the refreshed bf16 values go to every rank's replica of
// the flat parameter buffer (P.buf = flat_param on each rank) at [lo, lo+n).  With `mc` the store is
// one multimem.st that NVSwitch replicates.  A closing barrier tells the peers their replica is whole.
// ------------------------------------------------------------------------------------------------
// Element ranges of the bucket (absolute indices, half-open) that are exempt from weight decay: the biases and norm
// weights that sit between the matrices of a layer bucket.  A handful per bucket, passed by value.
constexpr int MAX_NODECAY = 16;
struct NoDecay {
  long long lo[MAX_NODECAY], hi[MAX_NODECAY];
  int n;
};

__global__ void __launch_bounds__(512)
adamw_bcast_kernel(Peers P, void* mc, long long lo, long long n, float* __restrict__ master,
                   const float* __restrict__ grad, float* __restrict__ m, float* __restrict__ v, float lr, float b1,
                   float b2, float eps, float wd, float bc1, float bc2_sqrt, const float* __restrict__ clip,
                   uint32_t* epoch_ctr, uint32_t* local_gate, int channel, int* status, const NoDecay nd) {
  const uint32_t epoch = *epoch_ctr + 1;
  const float gs = clip ? *clip : 1.f;
  const long long nvec = n / 8;
  for (long long q = blockIdx.x * (long long)blockDim.x + threadIdx.x; q < nvec; q += (long long)gridDim.x * blockDim.x) {
    float pv[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long long i = q * 8 + h * 4;
      const float4 g4 = *reinterpret_cast<const float4*>(grad + i);
      float4 m4 = *reinterpret_cast<const float4*>(m + i), v4 = *reinterpret_cast<const float4*>(v + i);
      float4 p4 = *reinterpret_cast<const float4*>(master + i);
      const float g[4] = {g4.x * gs, g4.y * gs, g4.z * gs, g4.w * gs};
      float* mm = reinterpret_cast<float*>(&m4);
      float* vv = reinterpret_cast<float*>(&v4);
      float* pp = reinterpret_cast<float*>(&p4);
      // decay applies unless the element lies in an exempt range (checked per element: a range may start mid-vector)
      float wdj[4] = {wd, wd, wd, wd};
      if (wd != 0.f) {
        for (int r = 0; r < nd.n; ++r) {
          const long long a0 = lo + i;
          if (a0 + 4 > nd.lo[r] && a0 < nd.hi[r]) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (a0 + j >= nd.lo[r] && a0 + j < nd.hi[r]) wdj[j] = 0.f;
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        mm[j] = mm[j] * b1 + (1.f - b1) * g[j];
        vv[j] = vv[j] * b2 + (1.f - b2) * g[j] * g[j];
        float p = pp[j];
        p -= lr * wdj[j] * p;
        p -= (lr / bc1) * mm[j] / (sqrtf(vv[j]) / bc2_sqrt + eps);
        pp[j] = p;
        pv[h * 4 + j] = p;
      }
      *reinterpret_cast<float4*>(m + i) = m4;
      *reinterpret_cast<float4*>(v + i) = v4;
      *reinterpret_cast<float4*>(master + i) = p4;
    }
    uint4 o;
    o.x = pack_bf16(pv[0], pv[1]);
    o.y = pack_bf16(pv[2], pv[3]);
    o.z = pack_bf16(pv[4], pv[5]);
    o.w = pack_bf16(pv[6], pv[7]);
    if (mc != nullptr) {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(mc) + lo + q * 8;
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(o.x)),
                   "f"(__uint_as_float(o.y)), "f"(__uint_as_float(o.z)), "f"(__uint_as_float(o.w))
                   : "memory");
    } else {
#pragma unroll
      for (int p = 0; p < MAX_PEERS; ++p)
        if (p < P.world) reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(P.buf[p]) + lo)[q] = o;
    }
  }
  // all of this grid's stores must be visible to the peers before the barrier word is released
  __threadfence_system();
  __shared__ unsigned last;
  __syncthreads();
  // every block arrives on the gate counter in the high half of local_gate's neighbour word
  if (threadIdx.x == 0) last = atomicAdd(local_gate + 1, 1u);
  __syncthreads();
  if (last == gridDim.x - 1) {  // the last block to finish runs the cross-GPU barrier on behalf of the grid
    if (threadIdx.x == 0) local_gate[1] = 0;
    __shared__ int ok_s;
    if (threadIdx.x == 0) ok_s = 1;
    __syncthreads();
    if (threadIdx.x < P.world) {
      st_release_sys(P.pad[threadIdx.x] + channel * MAX_PEERS + P.rank, epoch);
      const uint32_t* mine = P.pad[P.rank] + channel * MAX_PEERS + threadIdx.x;
      const uint64_t t0 = globaltimer_ns();
      while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
        if (globaltimer_ns() - t0 > kPeerWaitNs) {
          report_error(status, ERR_WAIT_TIMEOUT, 540, (int)threadIdx.x);
          break;
        }
        __nanosleep(64);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) *epoch_ctr = epoch;
  }
}

// ------------------------------------------------------------------------------------------------
// shard_allgather: every rank owns elements [rank*per, (rank+1)*per) of a bf16 buffer of world*per
// elements (P.buf = that buffer on each rank).  mode 0: pull the other shards from their owners;
// mode 1: push the own shard to everyone with multimem.st (mc = multicast mapping).
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512)
shard_allgather_kernel(Peers P, void* mc, long long per, uint32_t* epoch_ctr, uint32_t* local_gate, int channel,
                       int* status) {
  const uint32_t epoch = *epoch_ctr + 1;
  // entry barrier: the owners' shards are final (their producing kernels ran earlier on their streams)
  if (!peers_barrier(P, channel, epoch, local_gate, status, 560)) return;
  const long long nvec = per / 8;
  if (mc != nullptr) {
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(P.buf[P.rank]) + P.rank * per);
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(mc) + P.rank * per;
    for (long long q = blockIdx.x * (long long)blockDim.x + threadIdx.x; q < nvec; q += (long long)gridDim.x * blockDim.x) {
      const uint4 o = src[q];
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + q * 8),
                   "f"(__uint_as_float(o.x)), "f"(__uint_as_float(o.y)), "f"(__uint_as_float(o.z)),
                   "f"(__uint_as_float(o.w))
                   : "memory");
    }
  } else {
    uint4* mine = reinterpret_cast<uint4*>(P.buf[P.rank]);
    for (int s = 1; s < P.world; ++s) {
      const int owner = (P.rank + s) % P.world;  // staggered so the ranks do not all hit one owner at once
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(P.buf[owner]) + owner * per);
      uint4* dst = mine + owner * nvec;
      for (long long q = blockIdx.x * (long long)blockDim.x + threadIdx.x; q < nvec; q += (long long)gridDim.x * blockDim.x)
        dst[q] = src[q];
    }
  }
  __threadfence_system();
  __shared__ unsigned last;
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(local_gate + 1, 1u);
  __syncthreads();
  if (last == gridDim.x - 1) {
    if (threadIdx.x == 0) local_gate[1] = 0;
    // closing barrier (pushed data has landed everywhere / nobody overwrites a shard still being pulled)
    const uint32_t e2 = epoch + 1;
    if (threadIdx.x < P.world) {
      st_release_sys(P.pad[threadIdx.x] + channel * MAX_PEERS + P.rank, e2);
      const uint32_t* w = P.pad[P.rank] + channel * MAX_PEERS + threadIdx.x;
      const uint64_t t0 = globaltimer_ns();
      while ((int32_t)(ld_acquire_sys(w) - e2) < 0) {
        if (globaltimer_ns() - t0 > kPeerWaitNs) {
          report_error(status, ERR_WAIT_TIMEOUT, 580, (int)threadIdx.x);
          break;
        }
        __nanosleep(64);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) *epoch_ctr = e2;
  }
}

// ------------------------------------------------------------------------------------------------
// allreduce_add_rmsnorm (TP decode): res[T,H] += sum_p partial_p[T,H]; y = rmsnorm(res) * w.
// P.buf[p] = base of rank p's partial buffers (two buffers of T*H bf16, used alternately so a fast rank's
// next GEMM never overwrites a buffer a slow peer still reads).  One CTA per row; the sum runs in rank
// order on every rank, so all ranks compute bit-identical residual streams.
// ------------------------------------------------------------------------------------------------
template <int VPT>
__global__ void __launch_bounds__(256)
allreduce_add_rmsnorm_kernel(Peers P, long long buf_elems, __nv_bfloat16* __restrict__ res,
                             const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, int H, float eps,
                             uint32_t* epoch_ctr, uint32_t* local_gate, int channel, int* status) {
  const uint32_t epoch = *epoch_ctr + 1;
  if (!peers_barrier(P, channel, epoch, local_gate, status, 600)) return;
  const long long which = (long long)(epoch & 1u) * buf_elems;
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
      float acc[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16(au[j]); acc[2 * j] = f.x; acc[2 * j + 1] = f.y; }
      float part[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int p = 0; p < MAX_PEERS; ++p) {
        if (p < P.world) {
          const uint4 d = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(P.buf[p]) + which +
                                                        (size_t)row * H)[v];
          const uint32_t* du = reinterpret_cast<const uint32_t*>(&d);
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16(du[j]); part[2 * j] += f.x; part[2 * j + 1] += f.y; }
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // the summed block output is rounded to bf16 first (what an unfused all-reduce would hand over)
        const float2 s = unpack_bf16(pack_bf16(part[2 * j], part[2 * j + 1]));
        au[j] = pack_bf16(acc[2 * j] + s.x, acc[2 * j + 1] + s.y);
        const float2 r = unpack_bf16(au[j]);
        buf[i][2 * j] = r.x; buf[i][2 * j + 1] = r.y;
        ss += r.x * r.x + r.y * r.y;
      }
      xr[v] = a;
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
  if (grid_last_block(local_gate + 1) && threadIdx.x == 0) *epoch_ctr = epoch;
}

// ------------------------------------------------------------------------------------------------
// Consumer of the row-parallel decode GEMM that is fused with its all-reduce (decode_gemm.cu): every rank's GEMM
// CTAs have added their fp32 partial sums into `delta` of EVERY rank and then bumped `arrive` on every rank.
// This kernel waits (bounded) until `arrive` has reached `target` = ranks x CTAs per GEMM, then does
// res += bf16(delta), delta = 0, y = rmsnorm(res) * w.  The last CTA to finish takes `target` off the counter, so
// the counter never has to be cleared from the host and arrivals for the next use may already be coming in.
// One CTA per row; `done` is a zero-initialised word that the kernel leaves at zero.
// ------------------------------------------------------------------------------------------------
template <int VPT>
__global__ void __launch_bounds__(256)
add_rmsnorm_f32_wait_kernel(__nv_bfloat16* __restrict__ res, float* __restrict__ delta,
                            const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, int H, float eps,
                            uint32_t* arrive, uint32_t target, uint32_t* done, int* status) {
  __shared__ float red[8];
  __shared__ int ok_s;
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  if (tid == 0) {
    int ok = 1;
    const uint64_t t0 = globaltimer_ns();
    while (ld_acquire_sys(arrive) < target) {
      if (globaltimer_ns() - t0 > kPeerWaitNs) {
        report_error(status, ERR_WAIT_TIMEOUT, 610, (int)ld_acquire_sys(arrive));
        ok = 0;
        break;
      }
      __nanosleep(32);
    }
    ok_s = ok;
  }
  __syncthreads();
  if (!ok_s) return;
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
      const float4 d0 = __ldcg(dr + 2 * v), d1 = __ldcg(dr + 2 * v + 1);  // written by peers: read at L2
      dr[2 * v] = make_float4(0.f, 0.f, 0.f, 0.f);
      dr[2 * v + 1] = make_float4(0.f, 0.f, 0.f, 0.f);
      const float dv[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16(au[j]);
        // the block output is rounded to bf16 first (what an unfused GEMM + all-reduce would hand over)
        const float2 s = unpack_bf16(pack_bf16(dv[2 * j], dv[2 * j + 1]));
        au[j] = pack_bf16(f.x + s.x, f.y + s.y);
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
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(done, 1u) == gridDim.x - 1) {  // every CTA of this launch is past its wait
      *done = 0;
      atomicSub(arrive, target);
    }
  }
}

// Token agreement of a tensor-parallel decode group: rank 0's sampled tokens (and their log-probs) are the group's.
// Rank 0 stores them into every peer's mailbox and raises the peer's flag to the call's epoch; the other ranks wait
// (bounded) for their flag and copy the mailbox over their own samples.  With partial sums added in arrival order
// (atomics) the ranks' logits may differ in the last bit, so sampling on every rank from "identical" logits is not
// safe any more; one small message per step is.  mail[p] = rank p's mailbox (B ints then B floats), flag[p] its flag.
struct TokenSync {
  int* mail[MAX_PEERS];
  uint32_t* flag[MAX_PEERS];
  int rank, world;
};

__global__ void __launch_bounds__(256) tp_token_sync_kernel(TokenSync S, int* __restrict__ tok, float* __restrict__ logp,
                                                            int B, uint32_t* epoch_ctr, int* status) {
  __shared__ int ok_s;
  const uint32_t epoch = *epoch_ctr + 1;
  if (S.rank == 0) {
    for (int p = 1; p < S.world; ++p) {
      for (int i = threadIdx.x; i < B; i += blockDim.x) {
        S.mail[p][i] = tok[i];
        reinterpret_cast<float*>(S.mail[p] + B)[i] = logp[i];
      }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x > 0 && threadIdx.x < S.world) st_release_sys(S.flag[threadIdx.x], epoch);
  } else {
    if (threadIdx.x == 0) {
      int ok = 1;
      const uint64_t t0 = globaltimer_ns();
      while ((int32_t)(ld_acquire_sys(S.flag[S.rank]) - epoch) < 0) {
        if (globaltimer_ns() - t0 > kPeerWaitNs) {
          report_error(status, ERR_WAIT_TIMEOUT, 620, (int)epoch);
          ok = 0;
          break;
        }
        __nanosleep(32);
      }
      ok_s = ok;
    }
    __syncthreads();
    if (ok_s) {
      const int* mail = S.mail[S.rank];
      for (int i = threadIdx.x; i < B; i += blockDim.x) {
        tok[i] = __ldcg(mail + i);
        logp[i] = __ldcg(reinterpret_cast<const float*>(mail + B) + i);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *epoch_ctr = epoch;
}

// Self-test of the bounded-wait discipline: one thread polls a flag with a time budget, exactly like the peer
// waits above; when nothing sets the flag the kernel records ERR_WAIT_TIMEOUT and returns, and the context stays
// usable.  Used by the failure-detection test.
__global__ void bounded_wait_selftest_kernel(const uint32_t* flag, uint32_t expect, uint64_t budget_ns, int* status) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const uint64_t t0 = globaltimer_ns();
  while ((int32_t)(ld_acquire_sys(flag) - expect) < 0) {
    if (globaltimer_ns() - t0 > budget_ns) {
      report_error(status, ERR_WAIT_TIMEOUT, 999, (int)expect);
      return;
    }
    __nanosleep(64);
  }
}

// ------------------------------------------------------------------------------------------------
// shard_pull: dst[owner * per + i] = src_owner[i] for every owner (16-byte vectors, four in flight per thread); the
// owners are visited starting after this rank so that the ranks do not all read one owner at once.  No flags: the
// caller orders the launch after the point where the owners' slices became final.
// ------------------------------------------------------------------------------------------------
struct PullSrc {
  const uint4* src[MAX_PEERS];
};

__global__ void __launch_bounds__(512) shard_pull_kernel(PullSrc S, uint4* __restrict__ dst, long long nvec, int world,
                                                         int rank) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int s = 1; s <= world; ++s) {
    const int owner = (rank + s) % world;  // the own slice comes last
    const uint4* __restrict__ src = nullptr;
#pragma unroll
    for (int p = 0; p < MAX_PEERS; ++p)
      if (p == owner) src = S.src[p];  // static indices: the parameter struct stays in constant memory
    uint4* d = dst + owner * nvec;
    long long q = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    for (; q + 3 * stride < nvec; q += 4 * stride) {
      const uint4 a = src[q], b = src[q + stride], c = src[q + 2 * stride], e = src[q + 3 * stride];
      d[q] = a; d[q + stride] = b; d[q + 2 * stride] = c; d[q + 3 * stride] = e;
    }
    for (; q < nvec; q += stride) d[q] = src[q];
  }
}

// Trainer -> generator weight sync from sharded parameters: a list of contiguous ranges, each read from the rank that
// owns it (a peer mapping of the symmetric parameter arena, or local memory) and written into this rank's
// tensor-parallel weight buffers.  One CTA per range at a time, 16 bytes per thread and iteration.  The list is built
// once on the host (the layout of buckets and TP slices does not change during training).
struct CopyEntry {
  unsigned long long src, dst;
  unsigned long long bytes;  // multiple of 16; src and dst 16-byte aligned
};

__global__ void __launch_bounds__(256) copy_list_kernel(const CopyEntry* __restrict__ list, int n) {
  for (int e = blockIdx.x; e < n; e += gridDim.x) {
    const CopyEntry c = list[e];
    const uint4* s = reinterpret_cast<const uint4*>(c.src);
    uint4* d = reinterpret_cast<uint4*>(c.dst);
    const unsigned long long nv = c.bytes >> 4;
    for (unsigned long long v = threadIdx.x; v < nv; v += blockDim.x) d[v] = s[v];
  }
}

}  // namespace trlb

using namespace trlb;

static Peers make_peers(const unsigned long long* bufs, const unsigned long long* pads, int rank, int world) {
  Peers P;
  for (int i = 0; i < MAX_PEERS; ++i) {
    P.buf[i] = i < world ? reinterpret_cast<void*>(bufs[i]) : nullptr;
    P.pad[i] = i < world ? reinterpret_cast<uint32_t*>(pads[i]) : nullptr;
  }
  P.rank = rank;
  P.world = world;
  return P;
}

static int capped_grid(long long work_items, int threads) {
  long long g = (work_items + threads - 1) / threads;
  const int cap = trlb_host::sm_count();  // co-resident: blocks wait on block 0's barrier
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

// sync words: epoch_ctr (1 word) and local_gate (2 words) live in caller-provided device memory, zeroed once.
TRLB_API int trlb_rs_reduce(const unsigned long long* bufs, const unsigned long long* pads, int rank, int world,
                            const void* mc, int grad_is_bf16, long long lo, long long n, float* out, float* sumsq,
                            unsigned* epoch_ctr, unsigned* local_gate, int channel, int* status, cudaStream_t st) {
  if (world > MAX_PEERS || n % 8 != 0 || lo % 8 != 0) return -1;
  Peers P = make_peers(bufs, pads, rank, world);
  const int grid = capped_grid(n / 4, 512);
  if (grad_is_bf16)
    rs_reduce_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(P, nullptr, lo, n, out, sumsq, epoch_ctr, local_gate, channel, status, 0);
  else
    rs_reduce_kernel<float><<<grid, 512, 0, st>>>(P, mc, lo, n, out, sumsq, epoch_ctr, local_gate, channel, status, 0);
  return (int)cudaGetLastError();
}

// out[n] (fp32) += mean over ranks of grad[lo:lo+n] (bf16 or fp32 buffers read in place over peer loads).  The
// squared norm of the means of this call (not of the accumulator) is added to sumsq.  max_ctas bounds the grid so
// that the kernel can run beside a backward pass (0 = one CTA per SM).
TRLB_API int trlb_rs_reduce_accum(const unsigned long long* bufs, const unsigned long long* pads, int rank, int world,
                                  int grad_is_bf16, long long lo, long long n, float* out, float* sumsq,
                                  unsigned* epoch_ctr, unsigned* local_gate, int channel, int max_ctas, int* status,
                                  cudaStream_t st) {
  if (world > MAX_PEERS || n % 8 != 0 || lo % 8 != 0) return -1;
  Peers P = make_peers(bufs, pads, rank, world);
  int grid = capped_grid(n / 4, 512);
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grad_is_bf16)
    rs_reduce_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(P, nullptr, lo, n, out, sumsq, epoch_ctr, local_gate, channel, status, 1);
  else
    rs_reduce_kernel<float><<<grid, 512, 0, st>>>(P, nullptr, lo, n, out, sumsq, epoch_ctr, local_gate, channel, status, 1);
  return (int)cudaGetLastError();
}

TRLB_API int trlb_norm_allreduce(const unsigned long long* bufs, const unsigned long long* pads, int rank, int world,
                                 const float* my_sumsq, float max_norm, float* norm_out, float* clip_out,
                                 unsigned* epoch_ctr, unsigned* local_gate, int channel, int* status, cudaStream_t st) {
  if (world > MAX_PEERS) return -1;
  Peers P = make_peers(bufs, pads, rank, world);
  norm_allreduce_kernel<<<1, 32, 0, st>>>(P, my_sumsq, max_norm, norm_out, clip_out, epoch_ctr, local_gate, channel, status);
  return (int)cudaGetLastError();
}

TRLB_API int trlb_adamw_bcast(const unsigned long long* bufs, const unsigned long long* pads, int rank, int world, void* mc,
                              long long lo, long long n, float* master, const float* grad, float* m, float* v, int step,
                              float lr, float b1, float b2, float eps, float wd, const float* clip, unsigned* epoch_ctr,
                              unsigned* local_gate, int channel, int* status, const long long* nodecay, int n_nodecay,
                              cudaStream_t st) {
  // nodecay: n_nodecay pairs (lo, hi) of absolute element indices of the bucket that take no weight decay (host array)
  if (world > MAX_PEERS || n % 8 != 0 || lo % 8 != 0 || n_nodecay < 0 || n_nodecay > MAX_NODECAY) return -1;
  Peers P = make_peers(bufs, pads, rank, world);
  NoDecay nd = {};
  for (int r = 0; r < n_nodecay; ++r) {
    // keep only what intersects this rank's shard [lo, lo + n)
    const long long a = nodecay[2 * r], b = nodecay[2 * r + 1];
    if (b > lo && a < lo + n) { nd.lo[nd.n] = a; nd.hi[nd.n] = b; ++nd.n; }
  }
  const float bc1 = 1.f - powf(b1, (float)step), bc2s = sqrtf(1.f - powf(b2, (float)step));
  const int grid = capped_grid(n / 8, 512);
  adamw_bcast_kernel<<<grid, 512, 0, st>>>(P, mc, lo, n, master, grad, m, v, lr, b1, b2, eps, wd, bc1, bc2s, clip,
                                           epoch_ctr, local_gate, channel, status, nd);
  return (int)cudaGetLastError();
}

TRLB_API int trlb_shard_allgather(const unsigned long long* bufs, const unsigned long long* pads, int rank, int world,
                                  void* mc, long long per, unsigned* epoch_ctr, unsigned* local_gate, int channel,
                                  int* status, cudaStream_t st) {
  if (world > MAX_PEERS || per % 8 != 0) return -1;
  Peers P = make_peers(bufs, pads, rank, world);
  const int grid = capped_grid(per / 8, 512);
  shard_allgather_kernel<<<grid, 512, 0, st>>>(P, mc, per, epoch_ctr, local_gate, channel, status);
  return (int)cudaGetLastError();
}

TRLB_API int trlb_allreduce_add_rmsnorm(const unsigned long long* bufs, const unsigned long long* pads, int rank, int world,
                                        long long buf_elems, void* res, const void* w, void* y, int T, int H, float eps,
                                        unsigned* epoch_ctr, unsigned* local_gate, int channel, int* status,
                                        cudaStream_t st) {
  if (world > MAX_PEERS || H % 8 != 0 || H > 8192 || T > trlb_host::sm_count()) return -1;  // co-resident grid
  Peers P = make_peers(bufs, pads, rank, world);
  const int vpt = (H / 8 + 255) / 256;
  auto R = (__nv_bfloat16*)res; auto W = (const __nv_bfloat16*)w; auto Y = (__nv_bfloat16*)y;
  if (vpt <= 1) allreduce_add_rmsnorm_kernel<1><<<T, 256, 0, st>>>(P, buf_elems, R, W, Y, H, eps, epoch_ctr, local_gate, channel, status);
  else if (vpt <= 2) allreduce_add_rmsnorm_kernel<2><<<T, 256, 0, st>>>(P, buf_elems, R, W, Y, H, eps, epoch_ctr, local_gate, channel, status);
  else allreduce_add_rmsnorm_kernel<4><<<T, 256, 0, st>>>(P, buf_elems, R, W, Y, H, eps, epoch_ctr, local_gate, channel, status);
  return (int)cudaGetLastError();
}

// res[T,H] += bf16(delta32[T,H]) once `arrive` has reached `target`; delta32 is cleared, y = rmsnorm(res) * w and the
// last CTA subtracts `target` from `arrive` (see add_rmsnorm_f32_wait_kernel).  `done`: zero-initialised scratch word.
TRLB_API int trlb_add_rmsnorm_f32_wait(void* res, float* delta, const void* w, void* y, int T, int H, float eps,
                                       unsigned* arrive, unsigned target, unsigned* done, int* status, cudaStream_t st) {
  if (T == 0) return 0;
  if (H % 8 != 0 || H > 8192 || T > 4 * trlb_host::sm_count()) return -1;  // every CTA must become resident
  auto R = (__nv_bfloat16*)res; auto W = (const __nv_bfloat16*)w; auto Y = (__nv_bfloat16*)y;
  const int vpt = (H / 8 + 255) / 256;
  auto kern = vpt <= 1 ? add_rmsnorm_f32_wait_kernel<1>
                       : (vpt <= 2 ? add_rmsnorm_f32_wait_kernel<2> : add_rmsnorm_f32_wait_kernel<4>);
  return (int)trlb_host::launch_kernel(kern, dim3(T), dim3(256), 0, st, trlb_host::pdl_enabled(), R, delta, W, Y, H, eps,
                                       arrive, target, done, status);
}

// Rank 0's tok / logp (B entries each) become every rank's; mails[p] / flags[p] are rank p's mailbox (2 * B words)
// and flag word in symmetric memory; epoch_ctr is a local zero-initialised word.
TRLB_API int trlb_tp_token_sync(const unsigned long long* mails, const unsigned long long* flags, int rank, int world,
                                int* tok, float* logp, int B, unsigned* epoch_ctr, int* status, cudaStream_t st) {
  if (world < 2) return 0;
  if (world > MAX_PEERS) return -1;
  TokenSync S;
  for (int p = 0; p < MAX_PEERS; ++p) {
    S.mail[p] = p < world ? reinterpret_cast<int*>(mails[p]) : nullptr;
    S.flag[p] = p < world ? reinterpret_cast<uint32_t*>(flags[p]) : nullptr;
  }
  S.rank = rank; S.world = world;
  tp_token_sync_kernel<<<1, 256, 0, st>>>(S, tok, logp, B, epoch_ctr, status);
  return (int)cudaGetLastError();
}

TRLB_API int trlb_bounded_wait_selftest(const void* flag, unsigned expect, int budget_ms, int* status, cudaStream_t st) {
  if (budget_ms < 1 || budget_ms > 1000) return -160;  // the budget is what keeps this from being a hang
  bounded_wait_selftest_kernel<<<1, 32, 0, st>>>((const uint32_t*)flag, expect, (uint64_t)budget_ms * 1000000ull, status);
  return (int)cudaGetLastError();
}

// srcs[p]: rank p's slice (per elements of 2 bytes, 16-byte aligned, per a multiple of 8) as mapped by this rank;
// dst: local buffer of world * per elements.  ctas: grid size (it shares the GPU with the compute stream).
TRLB_API int trlb_shard_pull(const unsigned long long* srcs, int rank, int world, void* dst, long long per, int ctas,
                             cudaStream_t st) {
  if (world < 1 || world > MAX_PEERS || per % 8 != 0 || (reinterpret_cast<uintptr_t>(dst) & 15)) return -1;
  PullSrc S;
  for (int p = 0; p < MAX_PEERS; ++p) {
    S.src[p] = p < world ? reinterpret_cast<const uint4*>(srcs[p]) : nullptr;
    if (p < world && (srcs[p] & 15)) return -1;
  }
  if (ctas < 1) ctas = 32;
  if (ctas > 4 * trlb_host::sm_count()) ctas = 4 * trlb_host::sm_count();
  shard_pull_kernel<<<ctas, 512, 0, st>>>(S, (uint4*)dst, per / 8, world, rank);
  return (int)cudaGetLastError();
}

// list: device array of n {src, dst, bytes} triples (uint64 each).
TRLB_API int trlb_copy_list(const void* list, int n, cudaStream_t st) {
  if (n <= 0) return 0;
  int grid = n < 148 * 8 ? n : 148 * 8;
  copy_list_kernel<<<grid, 256, 0, st>>>((const CopyEntry*)list, n);
  return (int)cudaGetLastError();
}
