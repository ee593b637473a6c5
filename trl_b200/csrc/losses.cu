// Fused policy-optimisation losses (forward value, d/dlogp and metric sums in one pass).
//
//  grpo_loss   token-level clipped-ratio surrogate + k3 KL  (trl/trainer/grpo_trainer.py:3054-3150)
//  dpo_loss    masked per-sequence log-prob sums -> sigmoid preference loss, rewards, accuracy
//              (trl/trainer/dpo_trainer.py:1396-1435,1634-1635)
#include "common.cuh"

namespace trlb {

// stats layout (fp32, atomically accumulated; caller zeroes):
// [0] loss  [1] sum mask*kl  [2] sum mask*low_clipped  [3] sum mask*high_clipped  [4] sum mask
// [5] sum mask*ratio  [6] sum mask*min-branch-is-clipped  [7] sum mask*entropy (if given)
__global__ void __launch_bounds__(256)
grpo_loss_kernel(const float* __restrict__ logp, const float* __restrict__ old_logp, const float* __restrict__ ref_logp,
                 const float* __restrict__ adv, const float* __restrict__ mask, const float* __restrict__ row_scale,
                 const float* __restrict__ entropy, float* __restrict__ dlogp, float* __restrict__ tok_loss,
                 float* __restrict__ stats, int B, int T, float eps_low, float eps_high, float beta, float delta,
                 float grad_out) {
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const long long n = (long long)B * T;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(i / T);
    const float mk = mask[i];
    float d = 0.f, l = 0.f;
    if (mk != 0.f) {
      const float lp = logp[i];
      const float A = adv[b];
      const float ratio = old_logp ? __expf(lp - old_logp[i]) : 1.f;
      const float clipped = fminf(fmaxf(ratio, 1.f - eps_low), 1.f + eps_high);
      const float r1 = delta > 0.f ? fminf(ratio, delta) : ratio;
      const float s1 = r1 * A, s2 = clipped * A;
      const bool use1 = s1 <= s2;
      l = -(use1 ? s1 : s2);
      // d(-min)/dlogp: the unclipped branch carries gradient unless the two-sided cap is active
      float g = 0.f;
      if (use1) g = (delta > 0.f && ratio > delta) ? 0.f : -A * ratio;
      else g = (ratio >= 1.f - eps_low && ratio <= 1.f + eps_high) ? -A * ratio : 0.f;
      float kl = 0.f;
      if (ref_logp != nullptr && beta != 0.f) {
        const float dd = ref_logp[i] - lp;
        const float e = __expf(dd);
        kl = e - dd - 1.f;
        l += beta * kl;
        g += beta * (1.f - e);
      }
      const float w = mk * row_scale[b];
      d = g * w * grad_out;
      const bool lowc = (ratio < 1.f - eps_low) && (A < 0.f);
      const bool highc = (ratio > 1.f + eps_high) && (A > 0.f);
      acc[0] += l * w;
      acc[1] += mk * kl;
      acc[2] += lowc ? mk : 0.f;
      acc[3] += highc ? mk : 0.f;
      acc[4] += mk;
      acc[5] += mk * ratio;
      acc[6] += (lowc || highc) ? mk : 0.f;
      if (entropy) acc[7] += mk * entropy[i];
    }
    if (dlogp) dlogp[i] = d;
    if (tok_loss) tok_loss[i] = l;
  }
  __shared__ float sh[8][8];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float v = warp_sum(acc[k]);
    if (lane == 0) sh[k][wid] = v;
  }
  __syncthreads();
  if (threadIdx.x < 8) {
    float v = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) v += sh[threadIdx.x][w];
    atomicAdd(&stats[threadIdx.x], v);
  }
}

// One CTA per preference pair.  Sequences are rows of a packed token stream: sequence s covers
// tokens [cu[s], cu[s+1]); chosen = s in [0,P), rejected = s in [P,2P).
// out[pair*8 + ..]: 0 loss, 1 chosen reward, 2 rejected reward, 3 accuracy, 4 policy chosen logp,
// 5 policy rejected logp, 6 margin, 7 unused.
__global__ void __launch_bounds__(256)
dpo_loss_kernel(const float* __restrict__ pol, const float* __restrict__ ref, const float* __restrict__ mask,
                const int* __restrict__ cu, int P, float beta, float label_smoothing, float grad_scale,
                float* __restrict__ dpol, float* __restrict__ out) {
  const int pair = blockIdx.x;
  __shared__ float sh[4][8];
  __shared__ float coef[2];
  float sums[4] = {0.f, 0.f, 0.f, 0.f};
  for (int which = 0; which < 2; ++which) {
    const int s = pair + which * P;
    for (int t = cu[s] + threadIdx.x; t < cu[s + 1]; t += blockDim.x) {
      const float mk = mask[t];
      sums[which] += mk * pol[t];
      sums[2 + which] += mk * ref[t];
    }
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float v = warp_sum(sums[k]);
    if (lane == 0) sh[k][wid] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < 4; ++k)
      for (int w = 0; w < 8; ++w) tot[k] += sh[k][w];
    const float pc = tot[0], pr = tot[1], rc = tot[2], rr = tot[3];
    const float dlt = (pc - rc) - (pr - rr);
    const float x = beta * dlt;
    // -logsigmoid(x) = softplus(-x)
    const float sp_neg = fmaxf(-x, 0.f) + log1pf(__expf(-fabsf(x)));
    const float sp_pos = fmaxf(x, 0.f) + log1pf(__expf(-fabsf(x)));
    const float sig = 1.f / (1.f + __expf(-x));
    const float loss = (1.f - label_smoothing) * sp_neg + label_smoothing * sp_pos;
    // d loss / d delta
    const float dl = beta * (-(1.f - label_smoothing) * (1.f - sig) + label_smoothing * sig);
    coef[0] = dl * grad_scale;
    coef[1] = -dl * grad_scale;
    float* o = out + (size_t)pair * 8;
    o[0] = loss;
    o[1] = beta * (pc - rc);
    o[2] = beta * (pr - rr);
    o[3] = (o[1] > o[2]) ? 1.f : 0.f;
    o[4] = pc;
    o[5] = pr;
    o[6] = o[1] - o[2];
    o[7] = 0.f;
  }
  __syncthreads();
  if (dpol) {
    for (int which = 0; which < 2; ++which) {
      const int s = pair + which * P;
      const float c = coef[which];
      for (int t = cu[s] + threadIdx.x; t < cu[s + 1]; t += blockDim.x) dpol[t] = c * mask[t];
    }
  }
}

}  // namespace trlb

using namespace trlb;

TRLB_API int trlb_grpo_loss(const float* logp, const float* old_logp, const float* ref_logp, const float* adv,
                            const float* mask, const float* row_scale, const float* entropy, float* dlogp,
                            float* tok_loss, float* stats, int B, int T, float eps_low, float eps_high, float beta,
                            float delta, float grad_out, cudaStream_t st) {
  if (B == 0 || T == 0) return 0;
  long long n = (long long)B * T;
  int grid = (int)((n + 255) / 256);
  const int cap = trlb_host::sm_count() * 4;
  if (grid > cap) grid = cap;
  grpo_loss_kernel<<<grid, 256, 0, st>>>(logp, old_logp, ref_logp, adv, mask, row_scale, entropy, dlogp, tok_loss, stats,
                                        B, T, eps_low, eps_high, beta, delta, grad_out);
  return (int)cudaGetLastError();
}

TRLB_API int trlb_dpo_loss(const float* pol, const float* ref, const float* mask, const int* cu, int P, float beta,
                           float label_smoothing, float grad_scale, float* dpol, float* out, cudaStream_t st) {
  if (P == 0) return 0;
  dpo_loss_kernel<<<P, 256, 0, st>>>(pol, ref, mask, cu, P, beta, label_smoothing, grad_scale, dpol, out);
  return (int)cudaGetLastError();
}
