// RL math kernels: fused PPO token loss (forward + gradient + metrics in one pass),
// GAE reverse scan, group-normalised (GRPO) advantages, and the rollout sampler.
//
// Formulas follow verl/trainer/ppo/core_algos.py: GAE :214-262, GRPO :266-330,
// vanilla/dual-clip policy loss :1159-1250, kl_penalty :1841-1902. The reference
// runs these as many small torch launches (GAE is a Python loop over T).
#include "common.cuh"
#include "host_utils.h"

namespace vb {

__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_reduce_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? sh[lane] : 0.f;
  return warp_reduce_sum(t);
}

// metrics layout (sums over masked tokens):
// 0 pg_loss, 1 clipfrac, 2 ppo_kl, 3 clipfrac_lower, 4 kl_loss, 5 entropy, 6 mask count
struct PpoArgs {
  const float* logp;
  const float* old_logp;  // null => on-policy (old = logp detached)
  const float* adv;
  const float* mask;
  const float* ref_logp;  // null => no KL loss
  const float* entropy;   // null => no entropy bonus
  const float* is_weight; // null => no rollout importance weights
  float* d_logp;
  float* d_entropy;
  float* metrics;
  long long n;
  float clip_low, clip_high, clip_c, kl_coef, entropy_coeff, inv_denom;
  int kl_type;  // 0 kl(k1), 1 abs, 2 mse(k2), 3 low_var_kl(k3)
};

__global__ void ppo_loss_kernel(PpoArgs a) {
  __shared__ float sh[32];
  float acc[7] = {0, 0, 0, 0, 0, 0, 0};
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < a.n;
       i += (long long)gridDim.x * blockDim.x) {
    const float mk = a.mask[i];
    const float lp = a.logp[i];
    const float olp = a.old_logp ? a.old_logp[i] : lp;
    const float A = a.adv[i];
    const float w = a.is_weight ? a.is_weight[i] : 1.f;
    const float raw = lp - olp;
    const float nkl = fminf(fmaxf(raw, -20.f), 20.f);
    const bool in_range = (raw > -20.f) && (raw < 20.f);
    const float ratio = __expf(nkl);
    const float l1 = -A * ratio;
    const float rc = fminf(fmaxf(ratio, 1.f - a.clip_low), 1.f + a.clip_high);
    const float l2 = -A * rc;
    const float clip1 = fmaxf(l1, l2);
    const float l3 = -A * a.clip_c;
    const float clip2 = fminf(l3, clip1);
    const bool neg = A < 0.f;
    const float pg = neg ? clip2 : clip1;
    // gradient of pg wrt logp
    const float dl1 = in_range ? -A * ratio : 0.f;
    const bool ratio_clipped = (ratio < 1.f - a.clip_low) || (ratio > 1.f + a.clip_high);
    const float dl2 = ratio_clipped ? 0.f : dl1;
    float dclip1 = (l1 > l2) ? dl1 : ((l2 > l1) ? dl2 : 0.5f * (dl1 + dl2));
    float dpg = dclip1;
    if (neg) dpg = (l3 < clip1) ? 0.f : ((l3 > clip1) ? dclip1 : 0.5f * dclip1);
    float loss_grad = dpg * w;
    float kl = 0.f;
    if (a.ref_logp) {
      const float rlp = a.ref_logp[i];
      float dkl = 0.f;
      if (a.kl_type == 0) {
        kl = lp - rlp;
        dkl = 1.f;
      } else if (a.kl_type == 1) {
        kl = fabsf(lp - rlp);
        dkl = (lp > rlp) ? 1.f : ((lp < rlp) ? -1.f : 0.f);
      } else if (a.kl_type == 2) {
        kl = 0.5f * (lp - rlp) * (lp - rlp);
        dkl = lp - rlp;
      } else {
        const float draw = rlp - lp;
        const float d = fminf(fmaxf(draw, -20.f), 20.f);
        const float e = __expf(d);
        const float k3 = e - d - 1.f;
        kl = fminf(fmaxf(k3, -10.f), 10.f);
        const bool pass = (draw > -20.f) && (draw < 20.f) && (k3 > -10.f) && (k3 < 10.f);
        dkl = pass ? (1.f - e) : 0.f;
      }
      loss_grad += a.kl_coef * dkl;
    }
    a.d_logp[i] = loss_grad * mk * a.inv_denom;
    float ent = 0.f;
    if (a.entropy) {
      ent = a.entropy[i];
      if (a.d_entropy) a.d_entropy[i] = -a.entropy_coeff * mk * a.inv_denom;
    }
    acc[0] += pg * w * mk;
    acc[1] += (l2 > l1 ? 1.f : 0.f) * mk;
    acc[2] += -nkl * mk;
    acc[3] += ((clip1 > l3) && neg ? 1.f : 0.f) * mk;
    acc[4] += kl * mk;
    acc[5] += ent * mk;
    acc[6] += mk;
  }
#pragma unroll
  for (int j = 0; j < 7; ++j) {
    const float s = block_sum(acc[j], sh);
    if (threadIdx.x == 0) atomicAdd(a.metrics + j, s);
  }
}

// GAE: one thread per sequence, reverse scan with mask-aware carry
// (observation tokens keep nextvalues/lastgaelam: core_algos.py:214-262).
__global__ void gae_kernel(const float* __restrict__ rewards, const float* __restrict__ values,
                           const float* __restrict__ mask, float* __restrict__ adv, float* __restrict__ ret, int B,
                           int T, float gamma, float lam) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const long long off = (long long)b * T;
  float nextv = 0.f, last = 0.f;
  for (int t = T - 1; t >= 0; --t) {
    const float mk = mask[off + t];
    const float v = values[off + t];
    const float delta = rewards[off + t] + gamma * nextv - v;
    const float l_ = delta + gamma * lam * last;
    nextv = v * mk + (1.f - mk) * nextv;
    last = l_ * mk + (1.f - mk) * last;
    adv[off + t] = last;
    ret[off + t] = last + v;
  }
}

// GRPO: per-group mean / unbiased std of sequence scores; singleton groups use mean 0, std 1.
__global__ void group_stats_kernel(const float* __restrict__ scores, const int* __restrict__ gid, int B,
                                   float* __restrict__ gsum, float* __restrict__ gsq, float* __restrict__ gcnt) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const float s = scores[b];
  atomicAdd(gsum + gid[b], s);
  atomicAdd(gsq + gid[b], s * s);
  atomicAdd(gcnt + gid[b], 1.f);
}

__global__ void group_adv_kernel(const float* __restrict__ scores, const int* __restrict__ gid,
                                 const float* __restrict__ gsum, const float* __restrict__ gsq,
                                 const float* __restrict__ gcnt, const float* __restrict__ mask,
                                 float* __restrict__ adv, int B, int T, float eps, int norm_by_std) {
  const int b = blockIdx.x;
  const int g = gid[b];
  const float n = gcnt[g];
  float mean = 0.f, sd = 1.f;
  if (n > 1.5f) {
    mean = gsum[g] / n;
    const float var = fmaxf((gsq[g] - n * mean * mean) / (n - 1.f), 0.f);
    sd = sqrtf(var);
  }
  float a = scores[b] - mean;
  if (norm_by_std) a = a / (sd + eps);
  for (int t = threadIdx.x; t < T; t += blockDim.x) adv[(long long)b * T + t] = a * mask[(long long)b * T + t];
}

// ------------------------------- sampler -------------------------------------
__device__ __forceinline__ uint32_t mulhilo(uint32_t a, uint32_t b, uint32_t* hi) {
  const uint64_t p = (uint64_t)a * b;
  *hi = (uint32_t)(p >> 32);
  return (uint32_t)p;
}
// Philox-4x32-10, returns 4 x 32 random bits for (counter, key).
__device__ __forceinline__ uint4 philox(uint4 c, uint2 k) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, hi1;
    const uint32_t lo0 = mulhilo(0xD2511F53u, c.x, &hi0);
    const uint32_t lo1 = mulhilo(0xCD9E8D57u, c.z, &hi1);
    c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
    k.x += 0x9E3779B9u;
    k.y += 0xBB67AE85u;
  }
  return c;
}
__device__ __forceinline__ float u01(uint32_t x) { return ((float)(x >> 8) + 0.5f) * (1.f / 16777216.f); }

// Four consecutive logits starting at v0 (a multiple of 4) as floats; elements past V read as -inf. `vec` says that the
// row base is aligned for one 16-byte (fp32) / 8-byte (bf16) load.
__device__ __forceinline__ void load4_logits(const float* lg, bool vec, int v0, int V, float (&x)[4]) {
  if (vec && v0 + 3 < V) {
    const float4 t = *reinterpret_cast<const float4*>(lg + v0);
    x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = v0 + j < V ? lg[v0 + j] : -INFINITY;
  }
}
__device__ __forceinline__ void load4_logits(const __nv_bfloat16* lg, bool vec, int v0, int V, float (&x)[4]) {
  if (vec && v0 + 3 < V) {
    const uint2 t = *reinterpret_cast<const uint2*>(lg + v0);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = v0 + j < V ? __bfloat162float(lg[v0 + j]) : -INFINITY;
  }
}

// Unrestricted support (no top-k / top-p, or greedy): ONE pass over the row. Each thread keeps an online
// (max, sum of exp) pair and the Gumbel-max candidate of its elements; the argmax of logit / T + Gumbel noise needs no
// normaliser, and the log-prob of the winner is x - max - log(sum).
template <typename T>
__device__ __forceinline__ void sample_row_one_pass(const T* __restrict__ lg, int V, int row, float inv_t, bool greedy,
                                                    unsigned long long seed, unsigned long long st,
                                                    long long* __restrict__ token_out,
                                                    float* __restrict__ logprob_out) {
  __shared__ float sm_m[32], sm_z[32], sm_b[32];
  __shared__ int sm_i[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const bool vec = (reinterpret_cast<uintptr_t>(lg) & (4 * sizeof(T) - 1)) == 0;
  float m = -INFINITY, zs = 0.f, best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int v0 = threadIdx.x * 4; v0 < V; v0 += blockDim.x * 4) {
    float x[4];
    load4_logits(lg, vec, v0, V, x);
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] *= inv_t;
    const float gm = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
    if (gm > m) {
      zs *= __expf(m - gm);  // m = -inf: zs is still 0
      m = gm;
    }
    if (m > -INFINITY) zs += __expf(x[0] - m) + __expf(x[1] - m) + __expf(x[2] - m) + __expf(x[3] - m);
    uint32_t rr[4] = {0u, 0u, 0u, 0u};
    if (!greedy) {
      const uint4 rnd = philox(make_uint4((uint32_t)v0, (uint32_t)row, (uint32_t)st, (uint32_t)(st >> 32)),
                               make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
      rr[0] = rnd.x; rr[1] = rnd.y; rr[2] = rnd.z; rr[3] = rnd.w;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (v0 + j < V) {
        const float sc = greedy ? x[j] : x[j] - __logf(-__logf(u01(rr[j])));
        if (sc > best) {  // indices only grow inside a thread: ties keep the lowest
          best = sc;
          best_i = v0 + j;
        }
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), oz = __shfl_xor_sync(0xffffffffu, zs, o);
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    const float nm = fmaxf(m, om);
    zs = nm > -INFINITY ? zs * __expf(m - nm) + oz * __expf(om - nm) : 0.f;
    m = nm;
    if (ob > best || (ob == best && oi < best_i)) {
      best = ob;
      best_i = oi;
    }
  }
  if (lane == 0) {
    sm_m[warp] = m; sm_z[warp] = zs; sm_b[warp] = best; sm_i[warp] = best_i;
  }
  __syncthreads();
  if (warp == 0) {
    m = lane < nw ? sm_m[lane] : -INFINITY;
    zs = lane < nw ? sm_z[lane] : 0.f;
    best = lane < nw ? sm_b[lane] : -INFINITY;
    best_i = lane < nw ? sm_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o), oz = __shfl_xor_sync(0xffffffffu, zs, o);
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      const float nm = fmaxf(m, om);
      zs = nm > -INFINITY ? zs * __expf(m - nm) + oz * __expf(om - nm) : 0.f;
      m = nm;
      if (ob > best || (ob == best && oi < best_i)) {
        best = ob;
        best_i = oi;
      }
    }
    if (lane == 0) {
      const int tok = best_i < V ? best_i : 0;
      token_out[row] = tok;
      if (logprob_out) logprob_out[row] = ((float)lg[tok] * inv_t - m) - __logf(zs);
    }
  }
}

// One block per row. Gumbel-max sampling from softmax(logits / T) restricted by top-k / top-p
// (threshold found by bisection on the probability value), greedy when temperature == 0.
// Outputs the token and the log-prob of the sampled token under the *processed* distribution
// (temperature applied, restricted support renormalised), which is what the rollout reports
// as rollout_log_probs (vllm logprobs_mode=processed_logprobs in the reference config).
template <typename T>
__global__ void sample_kernel(const T* __restrict__ logits, long long row_stride, int V,
                              const float* __restrict__ temperature, const int* __restrict__ top_k,
                              const float* __restrict__ top_p, unsigned long long seed, const long long* __restrict__ step,
                              long long* __restrict__ token_out, float* __restrict__ logprob_out) {
  __shared__ float shf[32];
  __shared__ int shi[32];
  __shared__ float bc_f;
  __shared__ int bc_i;
  const int row = blockIdx.x;
  const T* lg = logits + (long long)row * row_stride;
  const float temp = temperature ? temperature[row] : 1.f;
  const bool greedy = temp <= 1e-6f;
  const float inv_t = greedy ? 1.f : 1.f / temp;
  const int k = top_k ? top_k[row] : -1;
  const float tp = top_p ? top_p[row] : 1.f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (greedy || !((k > 0 && k < V) || tp < 1.f)) {  // the same for every thread of the block
    sample_row_one_pass<T>(lg, V, row, inv_t, greedy, seed, step ? (unsigned long long)(*step) : 0ull, token_out,
                           logprob_out);
    return;
  }

  // pass 1: max
  float mx = -INFINITY;
  for (int v = threadIdx.x; v < V; v += blockDim.x) mx = fmaxf(mx, (float)lg[v] * inv_t);
  mx = warp_reduce_max(mx);
  if (lane == 0) shf[warp] = mx;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? shf[lane] : -INFINITY;
    t = warp_reduce_max(t);
    if (lane == 0) bc_f = t;
  }
  __syncthreads();
  mx = bc_f;
  __syncthreads();

  // pass 2: Z over full support
  float z = 0.f;
  for (int v = threadIdx.x; v < V; v += blockDim.x) z += __expf((float)lg[v] * inv_t - mx);
  z = block_sum(z, shf);
  if (threadIdx.x == 0) bc_f = z;
  __syncthreads();
  z = bc_f;
  __syncthreads();

  // support threshold on p = exp(x - mx) / z : keep tokens with p >= thr
  float thr = 0.f;
  const bool need_k = (k > 0 && k < V);
  const bool need_p = (tp < 1.f);
  if (!greedy && (need_k || need_p)) {
    // bisection on thr in [0, p_max]: count(p >= thr) and mass(p >= thr) are monotone
    // non-increasing in thr
    float lo = 0.f, hi = 1.f / z;  // p_max = exp(0)/z
    for (int it = 0; it < 30; ++it) {
      const float mid = 0.5f * (lo + hi);
      float cnt = 0.f, mass = 0.f;
      for (int v = threadIdx.x; v < V; v += blockDim.x) {
        const float p = __expf((float)lg[v] * inv_t - mx) / z;
        if (p >= mid) {
          cnt += 1.f;
          mass += p;
        }
      }
      cnt = block_sum(cnt, shf);
      mass = block_sum(mass, shf);
      if (threadIdx.x == 0) {
        // (top-k set) intersected with (top-p nucleus): thr = max(thr_k, thr_p), and
        // thr <= max(thr_k, thr_p) iff either constraint alone is still feasible at thr
        const bool feas = (need_k && cnt >= (float)k) || (need_p && mass >= tp);
        bc_i = feas ? 1 : 0;
      }
      __syncthreads();
      if (bc_i) lo = mid; else hi = mid;
      __syncthreads();
    }
    thr = lo;
  }

  // pass 3: Gumbel-max over the support, and the restricted normaliser
  unsigned long long st = step ? (unsigned long long)(*step) : 0ull;
  float best = -INFINITY;
  int best_i = 0;
  float zr = 0.f;
  for (int v0 = threadIdx.x * 4; v0 < V; v0 += blockDim.x * 4) {
    uint4 rnd = philox(make_uint4((uint32_t)v0, (uint32_t)row, (uint32_t)st, (uint32_t)(st >> 32)),
                       make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
    const uint32_t rr[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int v = v0 + j;
      if (v < V) {
        const float x = (float)lg[v] * inv_t - mx;
        const float e = __expf(x);
        if (e / z >= thr) {
          zr += e;
          const float g = greedy ? 0.f : -__logf(-__logf(u01(rr[j])));
          const float s = x + g;
          if (s > best) {
            best = s;
            best_i = v;
          }
        }
      }
    }
  }
  // block argmax (ties -> lowest index for determinism)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) {
      best = ob;
      best_i = oi;
    }
  }
  __syncthreads();
  if (lane == 0) {
    shf[warp] = best;
    shi[warp] = best_i;
  }
  __syncthreads();
  if (warp == 0) {
    float b = lane < nw ? shf[lane] : -INFINITY;
    int bi = lane < nw ? shi[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, b, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > b || (ob == b && oi < bi)) {
        b = ob;
        bi = oi;
      }
    }
    if (lane == 0) bc_i = bi;
  }
  __syncthreads();
  const int tok = bc_i;
  zr = block_sum(zr, shf);
  if (threadIdx.x == 0) {
    token_out[row] = tok;
    if (logprob_out) logprob_out[row] = ((float)lg[tok] * inv_t - mx) - __logf(zr);
  }
}

}  // namespace vb

using namespace vb;

extern "C" int vb_ppo_loss(const float* logp, const float* old_logp, const float* adv, const float* mask,
                           const float* ref_logp, const float* entropy, const float* is_weight, float* d_logp,
                           float* d_entropy, float* metrics, long long n, float clip_low, float clip_high,
                           float clip_c, float kl_coef, int kl_type, float entropy_coeff, float inv_denom,
                           cudaStream_t stream) {
  if (n <= 0) return 0;
  PpoArgs a{logp, old_logp, adv, mask, ref_logp, entropy, is_weight, d_logp, d_entropy, metrics, n,
            clip_low, clip_high, clip_c, kl_coef, entropy_coeff, inv_denom, kl_type};
  long long g = (n + 255) / 256;
  if (g > 148 * 4) g = 148 * 4;
  ppo_loss_kernel<<<(int)g, 256, 0, stream>>>(a);
  vb_count_launch();
  return (int)cudaGetLastError();
}

extern "C" int vb_gae(const float* rewards, const float* values, const float* mask, float* adv, float* ret, int B,
                      int T, float gamma, float lam, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  gae_kernel<<<(B + 63) / 64, 64, 0, stream>>>(rewards, values, mask, adv, ret, B, T, gamma, lam);
  vb_count_launch();
  return (int)cudaGetLastError();
}

// work: 3 * num_groups floats, zeroed by this call.
extern "C" int vb_grpo_adv(const float* scores, const int* gid, const float* mask, float* adv, float* work, int B,
                           int T, int num_groups, float eps, int norm_by_std, cudaStream_t stream) {
  if (B <= 0) return 0;
  VB_CUDA_CHECK(cudaMemsetAsync(work, 0, sizeof(float) * 3 * num_groups, stream));
  group_stats_kernel<<<(B + 127) / 128, 128, 0, stream>>>(scores, gid, B, work, work + num_groups,
                                                         work + 2 * num_groups);
  group_adv_kernel<<<B, 128, 0, stream>>>(scores, gid, work, work + num_groups, work + 2 * num_groups, mask, adv, B,
                                          T, eps, norm_by_std);
  vb_count_launch(2);
  return (int)cudaGetLastError();
}

// logits: [B, V] (dtype 0 = fp32, 1 = bf16), row_stride in elements. temperature/top_k/top_p are
// per-row device arrays (null = 1.0 / off / off). step is a device counter mixed into the RNG so a
// CUDA-graph replay draws fresh numbers when the caller increments it.
extern "C" int vb_sample(const void* logits, int dtype, long long row_stride, int B, int V, const float* temperature,
                         const int* top_k, const float* top_p, unsigned long long seed, const long long* step,
                         long long* token_out, float* logprob_out, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (dtype == 0)
    sample_kernel<float><<<B, 1024, 0, stream>>>((const float*)logits, row_stride, V, temperature, top_k, top_p, seed,
                                                 step, token_out, logprob_out);
  else
    sample_kernel<__nv_bfloat16><<<B, 1024, 0, stream>>>((const __nv_bfloat16*)logits, row_stride, V, temperature,
                                                         top_k, top_p, seed, step, token_out, logprob_out);
  vb_count_launch();
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------------------
// Decode-step chaining: the last kernel of a decode step turns the sampled tokens into the inputs of the next step,
// so that several steps (replays of one CUDA graph) run back to back without the host in between.
//   ring:   out_tok / out_lp [kmax, B] row *bpos receives this step's tokens / log-probs (-1 / 0 for rows that ended)
//   rows that are alive: a row ends when it samples `eos` (unless flags bit 0 = ignore eos) or reaches its length limit
//           (position + 2 >= limit: the sequence then holds `limit` tokens); it stops advancing and its cache slot
//           becomes -1, which the KV write skips
//   others: ids <- token, pos += 1, lens += 1, slot <- block_table[pos / block_size] * block_size + pos % block_size
//           (the host has reserved the pages of the whole burst before it started)
// One block; also advances the sampler's step counter and *bpos.
namespace vb {
__global__ void decode_advance_kernel(const long long* __restrict__ tok, const float* __restrict__ lp,
                                      long long* __restrict__ ids, long long* __restrict__ pos,
                                      long long* __restrict__ slots, int* __restrict__ lens,
                                      const int* __restrict__ bt, int mb, int block_size, const int* __restrict__ limit,
                                      int* __restrict__ alive, const int* __restrict__ flags, long long eos,
                                      long long* __restrict__ out_tok, float* __restrict__ out_lp, int* bpos,
                                      long long* sampler_step, int B, int kmax) {
  const int s = *bpos;
  __syncthreads();
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    const int a = alive[b];
    const long long t = tok[b];
    if (s >= 0 && s < kmax) {
      out_tok[(long long)s * B + b] = a ? t : -1;
      out_lp[(long long)s * B + b] = a ? lp[b] : 0.f;
    }
    if (a) {
      // lens[b] counts the tokens in the cache after this step: the token just processed has index lens - 1. The
      // RoPE position may differ from the token index (multimodal RoPE offsets text after images), so slots and the
      // length limit follow the index and the position just advances by one.
      const long long ti = (long long)lens[b] - 1;
      const bool done = (((flags[b] & 1) == 0) && t == eos) || (ti + 2 >= (long long)limit[b]);
      if (done) {
        alive[b] = 0;
        slots[b] = -1;
      } else {
        const long long ni = ti + 1;
        const int blk = (int)(ni / block_size);
        ids[b] = t;
        pos[b] += 1;
        lens[b] += 1;
        slots[b] = blk < mb ? (long long)bt[(long long)b * mb + blk] * block_size + (ni % block_size) : -1;
        if (blk >= mb) alive[b] = 0;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *bpos = s + 1;
    if (sampler_step != nullptr) *sampler_step += 1;
  }
}
}  // namespace vb

extern "C" int vb_decode_advance(const long long* tok, const float* lp, long long* ids, long long* pos, long long* slots,
                                 int* lens, const int* bt, int mb, int block_size, const int* limit, int* alive,
                                 const int* flags, long long eos, long long* out_tok, float* out_lp, int* bpos,
                                 long long* sampler_step, int B, int kmax, cudaStream_t stream) {
  if (B <= 0 || kmax <= 0 || block_size <= 0) return -3;
  vb::decode_advance_kernel<<<1, 256, 0, stream>>>(tok, lp, ids, pos, slots, lens, bt, mb, block_size, limit, alive, flags,
                                                   eos, out_tok, out_lp, bpos, sampler_step, B, kmax);
  vb_count_launch();
  return (int)cudaGetLastError();
}
