// Memory-bound model kernels: RMSNorm (with fused residual add), rotary embedding,
// SwiGLU, embedding gather/scatter, fused AdamW on flat shards, squared-norm reduction.
// All use 16-byte vector accesses; bf16 storage, fp32 math.
//
// These replace what the reference gets from HF eager / liger / apex
// (verl/models/llama/megatron/layers/parallel_rmsnorm.py:40-49, parallel_mlp.py) and
// torch.optim.AdamW + clip_grad_norm_ (verl/workers/actor/dp_actor.py:391-415).
#include "common.cuh"
#include "host_utils.h"

namespace vb {

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  bf16x8 t = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x = __bfloat1622float2(t.v[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  bf16x8 t;
#pragma unroll
  for (int i = 0; i < 4; ++i) t.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = t;
}

__device__ __forceinline__ float block_reduce_sum(float v, float* sh) {
  v = warp_reduce_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? sh[lane] : 0.f;
  t = warp_reduce_sum(t);
  return t;
}

// ------------------------------- RMSNorm ------------------------------------
// y = (x [+ res]) * rstd * w ; optionally writes the pre-norm sum to res_out.
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out, int H,
                                   float eps) {
  __shared__ float sh[32];
  pdl_trigger();
  pdl_wait();
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * H;
  const int nvec = H >> 3;
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    load8(xr + v * 8, f);
    if (res) {
      float g[8];
      load8(res + row * H + v * 8, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += g[i];
      if (res_out) {
        store8(res_out + row * H + v * 8, f);
        // re-round so the norm sees exactly what later layers will read
        load8(res_out + row * H + v * 8, f);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = block_reduce_sum(ss, sh);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  const __nv_bfloat16* src = (res && res_out) ? (res_out + row * H) : xr;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8], wv[8];
    load8(src + v * 8, f);
    if (res && !res_out) {
      float g[8];
      load8(res + row * H + v * 8, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += g[i];
    }
    load8(w + v * 8, wv);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * wv[i];
    store8(y + row * H + v * 8, f);
  }
}

// dx = rstd * (g - xhat * mean(g * xhat)), g = dy * w ; optionally dx += dres (gradient
// arriving through the residual path). dw partial sums go to dw_partial[gridDim.x, H].
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                                   float* __restrict__ dw_partial, int rows, int H) {
  extern __shared__ float dw_acc[];  // [H]
  __shared__ float sh[32];
  const int nvec = H >> 3;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dw_acc[i] = 0.f;
  __syncthreads();
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rs = rstd[row];
    float dot = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float fx[8], fdy[8], fw[8];
      load8(x + row * H + v * 8, fx);
      load8(dy + row * H + v * 8, fdy);
      load8(w + v * 8, fw);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = fx[i] * rs;
        dot += fdy[i] * fw[i] * xh;
        dw_acc[v * 8 + i] += fdy[i] * xh;
      }
    }
    dot = block_reduce_sum(dot, sh) / H;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float fx[8], fdy[8], fw[8], o[8];
      load8(x + row * H + v * 8, fx);
      load8(dy + row * H + v * 8, fdy);
      load8(w + v * 8, fw);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = rs * (fdy[i] * fw[i] - fx[i] * rs * dot);
      if (dres) {
        float fr[8];
        load8(dres + row * H + v * 8, fr);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += fr[i];
      }
      store8(dx + row * H + v * 8, o);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H; i += blockDim.x) dw_partial[(long long)blockIdx.x * H + i] = dw_acc[i];
}

__global__ void colsum_kernel(const float* __restrict__ partial, int nparts, int H, float* __restrict__ out,
                              int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int i = 0; i < nparts; ++i) s += partial[(long long)i * H + c];
  out[c] = accumulate ? out[c] + s : s;
}

// ------------------------------- RoPE ----------------------------------------
// In-place rotate-half rotary embedding on packed q [T, Hq, D] and k [T, Hk, D]
// (row strides given in elements). cos/sin tables are [max_pos, D/2] fp32.
// sign = +1 forward, -1 backward (transpose of the rotation).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k, long long q_stride,
                            long long k_stride, const long long* __restrict__ pos, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, int T, int Hq, int Hk, int D, float sign, int mrope_s0,
                            int mrope_s1) {
  // multimodal rotary embedding (mrope_s0 > 0): pos is [3, T] (temporal, height, width); rotary frequency j takes the
  // position of axis 0 for j < s0, of axis 1 for j < s0 + s1, of axis 2 above (sections are multiples of 8, so the 8
  // frequencies of one thread share an axis)
  pdl_trigger();
  pdl_wait();
  const int half = D >> 1;
  const int vec_per_head = half >> 3;
  const long long total = (long long)T * (Hq + Hk) * vec_per_head;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int v = idx % vec_per_head;
    const long long th = idx / vec_per_head;
    const int h = th % (Hq + Hk);
    const long long t = th / (Hq + Hk);
    __nv_bfloat16* base = (h < Hq) ? (q + t * q_stride + (long long)h * D) : (k + t * k_stride + (long long)(h - Hq) * D);
    long long p;
    if (mrope_s0 > 0) {
      const int j = v * 8;
      const int axis = j < mrope_s0 ? 0 : (j < mrope_s0 + mrope_s1 ? 1 : 2);
      p = pos[(long long)axis * T + t];
    } else {
      p = pos[t];
    }
    const float* c = cos_t + p * half + v * 8;
    const float* s = sin_t + p * half + v * 8;
    float a[8], b[8];
    load8(base + v * 8, a);
    load8(base + half + v * 8, b);
    float oa[8], ob[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float cs = c[i], sn = s[i] * sign;
      oa[i] = a[i] * cs - b[i] * sn;
      ob[i] = b[i] * cs + a[i] * sn;
    }
    store8(base + v * 8, oa);
    store8(base + half + v * 8, ob);
  }
}

// ------------------------------- SwiGLU --------------------------------------
// gu: [T, 2I] (gate | up), out: [T, I]
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long long T,
                                  int I) {
  pdl_trigger();
  pdl_wait();
  const int nvec = I >> 3;
  const long long total = T * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int v = idx % nvec;
    float g[8], u[8], o[8];
    load8(gu + t * 2 * I + v * 8, g);
    load8(gu + t * 2 * I + I + v * 8, u);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
    store8(out + t * I + v * 8, o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int I) {
  const int nvec = I >> 3;
  const long long total = T * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int v = idx % nvec;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + t * 2 * I + v * 8, g);
    load8(gu + t * 2 * I + I + v * 8, u);
    load8(dout + t * I + v * 8, d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sg = 1.f / (1.f + __expf(-g[i]));
      const float silu = g[i] * sg;
      dg[i] = d[i] * u[i] * (sg + silu * (1.f - sg));
      du[i] = d[i] * silu;
    }
    store8(dgu + t * 2 * I + v * 8, dg);
    store8(dgu + t * 2 * I + I + v * 8, du);
  }
}

// ------------------------------- Embedding -----------------------------------
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ w,
                                     __nv_bfloat16* __restrict__ out, long long T, int H) {
  const int nvec = H >> 3;
  const long long total = T * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int v = idx % nvec;
    *reinterpret_cast<uint4*>(out + t * H + v * 8) = *reinterpret_cast<const uint4*>(w + ids[t] * H + v * 8);
  }
}

// dW[ids[t], :] += dy[t, :] into an fp32 gradient buffer.
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dy,
                                     float* __restrict__ dw, long long T, int H) {
  const int nvec = H >> 3;
  const long long total = T * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int v = idx % nvec;
    float f[8];
    load8(dy + t * H + v * 8, f);
    float* dst = dw + ids[t] * H + v * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) atomicAdd(dst + i, f[i]);
  }
}

// ------------------------------- AdamW ---------------------------------------
// Flat-shard AdamW with fp32 master weights; writes the bf16 working copy in the same pass.
//   grad is fp32 (grad_bf16 == 0) or bf16. scale_ptr (device) multiplies the gradient
//   (clip coefficient and/or 1/world); skip_ptr (device) != 0 leaves everything unchanged
//   (non-finite gradient norm: verl/workers/actor/dp_actor.py:410-412).
__global__ void adamw_kernel(float* __restrict__ p32, const void* __restrict__ grad, int grad_bf16,
                             float* __restrict__ m, float* __restrict__ v, __nv_bfloat16* __restrict__ p16,
                             long long n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                             const float* __restrict__ scale_ptr, const int* __restrict__ skip_ptr) {
  if (skip_ptr && *skip_ptr) return;
  const float gs = scale_ptr ? *scale_ptr : 1.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float g = grad_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(grad)[i])
                        : reinterpret_cast<const float*>(grad)[i];
    g *= gs;
    float p = p32[i];
    float mi = m[i] * b1 + (1.f - b1) * g;
    float vi = v[i] * b2 + (1.f - b2) * g * g;
    m[i] = mi;
    v[i] = vi;
    p = p * (1.f - lr * wd);
    p -= lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    p32[i] = p;
    if (p16) p16[i] = __float2bfloat16(p);
  }
}

// out[0] += sum(x^2)  (fp32 or bf16 input)
__global__ void sumsq_kernel(const void* __restrict__ x, int is_bf16, long long n, float* __restrict__ out) {
  __shared__ float sh[32];
  float s = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float f = is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i])
                            : reinterpret_cast<const float*>(x)[i];
    s += f * f;
  }
  s = block_reduce_sum(s, sh);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

// scale_out = min(1, max_norm / (sqrt(sumsq) + 1e-6)); skip_out = !isfinite(norm); norm_out = norm
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float max_norm, float* __restrict__ scale_out,
                                 int* __restrict__ skip_out, float* __restrict__ norm_out, float extra_scale) {
  const float norm = sqrtf(*sumsq) * extra_scale;
  const bool finite = isfinite(norm);
  float c = 1.f;
  if (max_norm > 0.f && finite) c = fminf(1.f, max_norm / (norm + 1e-6f));
  *scale_out = c * extra_scale;
  *skip_out = finite ? 0 : 1;
  *norm_out = norm;
}

// bf16 <- fp32 cast (flat), and fp32 <- bf16
__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16(src[i]);
}

static inline int grid_for(long long work, int block, int max_blocks) {
  long long g = (work + block - 1) / block;
  if (g > max_blocks) g = max_blocks;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace vb

using namespace vb;

extern "C" int vb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out, float* rstd,
                              long long rows, int H, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H & 7) return -3;
  const int threads = H >= 4096 ? 512 : 256;
  cudaError_t e = vb_launch_pdl(rmsnorm_fwd_kernel, dim3((unsigned)rows), dim3(threads), 0, stream, 1,
                                (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w,
                                (__nv_bfloat16*)y, (__nv_bfloat16*)res_out, rstd, H, eps);
  vb_count_launch();
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// Number of partial rows the backward uses; dw_partial must hold that many rows of H floats.
extern "C" int vb_rmsnorm_bwd_parts(long long rows) {
  const int g = 6 * vb_num_sms();  // six resident blocks per SM: 75 % of the warp slots (two left the loads starved)
  return rows < g ? (int)rows : g;
}

extern "C" int vb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                              void* dx, float* dw_partial, float* dw, int dw_accumulate, long long rows, int H,
                              cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H & 7) return -3;
  const int parts = vb_rmsnorm_bwd_parts(rows);
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 48 * 1024) {
    VB_CUDA_CHECK(cudaFuncSetAttribute(rmsnorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  rmsnorm_bwd_kernel<<<parts, 256, smem, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                  (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres,
                                                  (__nv_bfloat16*)dx, dw_partial, (int)rows, H);
  colsum_kernel<<<(H + 255) / 256, 256, 0, stream>>>(dw_partial, parts, H, dw, dw_accumulate);
  vb_count_launch(2);
  return (int)cudaGetLastError();
}

static int rope_launch(void* q, void* k, long long q_stride, long long k_stride, const long long* pos, const float* cos_t,
                       const float* sin_t, int T, int Hq, int Hk, int D, int backward, int s0, int s1, cudaStream_t stream);

extern "C" int vb_rope(void* q, void* k, long long q_stride, long long k_stride, const long long* pos,
                       const float* cos_t, const float* sin_t, int T, int Hq, int Hk, int D, int backward,
                       cudaStream_t stream) {
  return rope_launch(q, k, q_stride, k_stride, pos, cos_t, sin_t, T, Hq, Hk, D, backward, 0, 0, stream);
}

// Multimodal RoPE: pos is [3, T]; s0 / s1 = number of rotary frequencies (of D / 2) that follow the temporal / height
// positions (the rest follow the width positions); both multiples of 8.
extern "C" int vb_mrope(void* q, void* k, long long q_stride, long long k_stride, const long long* pos3,
                        const float* cos_t, const float* sin_t, int T, int Hq, int Hk, int D, int s0, int s1, int backward,
                        cudaStream_t stream) {
  if (s0 <= 0 || s1 < 0 || (s0 & 7) || (s1 & 7) || s0 + s1 > D / 2) return -3;
  return rope_launch(q, k, q_stride, k_stride, pos3, cos_t, sin_t, T, Hq, Hk, D, backward, s0, s1, stream);
}

static int rope_launch(void* q, void* k, long long q_stride, long long k_stride, const long long* pos, const float* cos_t,
                       const float* sin_t, int T, int Hq, int Hk, int D, int backward, int s0, int s1, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D & 15) return -3;
  const long long total = (long long)T * (Hq + Hk) * (D / 16);
  cudaError_t e = vb_launch_pdl(rope_kernel, dim3(grid_for(total, 256, 148 * 16)), dim3(256), 0, stream, 1,
                                (__nv_bfloat16*)q, (__nv_bfloat16*)k, q_stride, k_stride, pos, cos_t, sin_t, T, Hq, Hk,
                                D, backward ? -1.f : 1.f, s0, s1);
  vb_count_launch();
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

extern "C" int vb_swiglu_fwd(const void* gu, void* out, long long T, int I, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (I & 7) return -3;
  cudaError_t e = vb_launch_pdl(swiglu_fwd_kernel, dim3(grid_for(T * (I / 8), 256, 148 * 16)), dim3(256), 0, stream, 1,
                                (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, I);
  vb_count_launch();
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

extern "C" int vb_swiglu_bwd(const void* gu, const void* dout, void* dgu, long long T, int I, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (I & 7) return -3;
  swiglu_bwd_kernel<<<grid_for(T * (I / 8), 256, 148 * 16), 256, 0, stream>>>(
      (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dgu, T, I);
  vb_count_launch();
  return (int)cudaGetLastError();
}

extern "C" int vb_embedding_fwd(const long long* ids, const void* w, void* out, long long T, int H,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H & 7) return -3;
  embedding_fwd_kernel<<<grid_for(T * (H / 8), 256, 148 * 16), 256, 0, stream>>>(ids, (const __nv_bfloat16*)w,
                                                                                 (__nv_bfloat16*)out, T, H);
  vb_count_launch();
  return (int)cudaGetLastError();
}

extern "C" int vb_embedding_bwd(const long long* ids, const void* dy, float* dw, long long T, int H,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H & 7) return -3;
  embedding_bwd_kernel<<<grid_for(T * (H / 8), 256, 148 * 16), 256, 0, stream>>>(ids, (const __nv_bfloat16*)dy, dw,
                                                                                 T, H);
  vb_count_launch();
  return (int)cudaGetLastError();
}

extern "C" int vb_adamw(float* p32, const void* grad, int grad_bf16, float* m, float* v, void* p16, long long n,
                        float lr, float b1, float b2, float eps, float wd, int step, const float* scale_ptr,
                        const int* skip_ptr, cudaStream_t stream) {
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(b1, (float)step);
  const float bc2 = 1.f - powf(b2, (float)step);
  adamw_kernel<<<grid_for(n, 256, 148 * 16), 256, 0, stream>>>(p32, grad, grad_bf16, m, v, (__nv_bfloat16*)p16, n, lr,
                                                               b1, b2, eps, wd, bc1, bc2, scale_ptr, skip_ptr);
  vb_count_launch();
  return (int)cudaGetLastError();
}

extern "C" int vb_sumsq(const void* x, int is_bf16, long long n, float* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  sumsq_kernel<<<grid_for(n, 256, 148 * 8), 256, 0, stream>>>(x, is_bf16, n, out);
  vb_count_launch();
  return (int)cudaGetLastError();
}

extern "C" int vb_clip_coef(const float* sumsq, float max_norm, float extra_scale, float* scale_out, int* skip_out,
                            float* norm_out, cudaStream_t stream) {
  clip_coef_kernel<<<1, 1, 0, stream>>>(sumsq, max_norm, scale_out, skip_out, norm_out, extra_scale);
  vb_count_launch();
  return (int)cudaGetLastError();
}

extern "C" int vb_cast_f32_bf16(const float* src, void* dst, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for(n, 256, 148 * 16), 256, 0, stream>>>(src, (__nv_bfloat16*)dst, n);
  vb_count_launch();
  return (int)cudaGetLastError();
}
