// Paged-KV decode attention and KV-cache writes for the native rollout engine.
// These take the place of the vLLM attention backends the reference calls through
// verl/workers/rollout/vllm_rollout/vllm_async_server.py:445-547.
//
// Cache layout (K and V each): [num_blocks, Hk, block_size, D] bf16, so all keys of one
// KV head inside a page are contiguous.
//
// Decode kernel: one CTA per (sequence, KV head, split). The CTA serves all G = Hq/Hk query
// heads of the group, so each K/V byte is read once per group. Per 128-key chunk:
//   phase 1: thread t scores key t against the G query vectors (q in shared memory)
//   phase 2: thread (pair, part) accumulates P.V for one pair of output dims over a slice of keys
// Online softmax across chunks; splits are merged by a second small kernel.
#include "common.cuh"
#include "host_utils.h"

namespace vb {

constexpr int CHUNK = 128;
constexpr int GMAX = 8;

template <int D>
__global__ void __launch_bounds__(128)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride,  // [B, Hq, D], stride per seq
                    const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                    const int* __restrict__ block_table, int max_blocks, const int* __restrict__ seq_lens,
                    int Hq, int Hk, int block_size, float scale, int num_splits,
                    __nv_bfloat16* __restrict__ out, long long out_stride,  // [B, Hq, D]
                    float* __restrict__ o_part,   // [B, Hq, S, D]
                    float* __restrict__ ml_part)  // [B, Hq, S, 2]
{
  constexpr int PAIRS = D / 2;
  constexpr int KPARTS = 128 / PAIRS;
  const int b = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
  const int G = Hq / Hk;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seq_len = seq_lens[b];

  __shared__ float q_s[GMAX][D];
  __shared__ float s_s[GMAX][CHUNK];
  __shared__ long long row_off[CHUNK];
  __shared__ float red[GMAX][4];
  __shared__ float alpha_s[GMAX];
  __shared__ float o_s[KPARTS][GMAX][D];

  for (int i = tid; i < G * D; i += 128) {
    const int g = i / D, d = i % D;
    q_s[g][d] = __bfloat162float(q[(long long)b * q_stride + (long long)(h * G + g) * D + d]) * scale;
  }
  // key range of this split (chunk aligned)
  const int chunks_total = (seq_len + CHUNK - 1) / CHUNK;
  const int chunks_per_split = (chunks_total + num_splits - 1) / num_splits;
  const int c_begin = split * chunks_per_split;
  const int c_end = min(chunks_total, c_begin + chunks_per_split);

  float m_run[GMAX], l_run[GMAX];
  float o_acc[GMAX][2];
#pragma unroll
  for (int g = 0; g < GMAX; ++g) {
    m_run[g] = -INFINITY;
    l_run[g] = 0.f;
    o_acc[g][0] = o_acc[g][1] = 0.f;
  }
  const int pair = tid % PAIRS, part = tid / PAIRS;
  __syncthreads();

  for (int c = c_begin; c < c_end; ++c) {
    const int key = c * CHUNK + tid;
    const bool valid = key < seq_len;
    float sc[GMAX];
#pragma unroll
    for (int g = 0; g < GMAX; ++g) sc[g] = 0.f;
    long long off = 0;
    if (valid) {
      const int blk = block_table[(long long)b * max_blocks + key / block_size];
      off = (((long long)blk * Hk + h) * block_size + (key % block_size)) * D;
      const uint4* kp = reinterpret_cast<const uint4*>(kc + off);
#pragma unroll 4
      for (int j = 0; j < D / 8; ++j) {
        const uint4 raw = kp[j];
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float kf[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h2[i]);
          kf[2 * i] = f.x;
          kf[2 * i + 1] = f.y;
        }
#pragma unroll
        for (int g = 0; g < GMAX; ++g) {
          if (g < G) {
            const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][j * 8]);
            const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][j * 8 + 4]);
            sc[g] += qa.x * kf[0] + qa.y * kf[1] + qa.z * kf[2] + qa.w * kf[3] + qb.x * kf[4] + qb.y * kf[5] +
                     qb.z * kf[6] + qb.w * kf[7];
          }
        }
      }
    }
    row_off[tid] = off;
    // chunk max per head
#pragma unroll
    for (int g = 0; g < GMAX; ++g) {
      if (g < G) {
        const float v = valid ? sc[g] : -INFINITY;
        sc[g] = v;
        const float wm = warp_reduce_max(v);
        if (lane == 0) red[g][warp] = wm;
      }
    }
    __syncthreads();
    float psum[GMAX];
#pragma unroll
    for (int g = 0; g < GMAX; ++g) {
      if (g < G) {
        const float cm = fmaxf(fmaxf(red[g][0], red[g][1]), fmaxf(red[g][2], red[g][3]));
        const float nm = fmaxf(m_run[g], cm);
        const float p = valid ? __expf(sc[g] - nm) : 0.f;
        s_s[g][tid] = p;
        psum[g] = warp_reduce_sum(p);
        const float alpha = __expf(m_run[g] - nm);
        if (tid == 0) alpha_s[g] = alpha;
        l_run[g] *= alpha;
        m_run[g] = nm;
      }
    }
    __syncthreads();  // red[] consumed by everyone, s_s/alpha_s visible
#pragma unroll
    for (int g = 0; g < GMAX; ++g)
      if (g < G && lane == 0) red[g][warp] = psum[g];
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GMAX; ++g) {
      if (g < G) {
        l_run[g] += red[g][0] + red[g][1] + red[g][2] + red[g][3];
        const float al = alpha_s[g];
        o_acc[g][0] *= al;
        o_acc[g][1] *= al;
      }
    }
    // phase 2: P.V
    const int nkeys = min(CHUNK, seq_len - c * CHUNK);
    for (int j = part; j < nkeys; j += KPARTS) {
      const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(vc + row_off[j] + 2 * pair);
      const float2 vf = __bfloat1622float2(v2);
#pragma unroll
      for (int g = 0; g < GMAX; ++g) {
        if (g < G) {
          const float p = s_s[g][j];
          o_acc[g][0] += p * vf.x;
          o_acc[g][1] += p * vf.y;
        }
      }
    }
    __syncthreads();  // before the next chunk overwrites s_s / row_off / red
  }

  // combine key-slices
#pragma unroll
  for (int g = 0; g < GMAX; ++g) {
    if (g < G) {
      o_s[part][g][2 * pair] = o_acc[g][0];
      o_s[part][g][2 * pair + 1] = o_acc[g][1];
    }
  }
  __syncthreads();
  for (int i = tid; i < G * D; i += 128) {
    const int g = i / D, d = i % D;
    float o = 0.f;
#pragma unroll
    for (int pt = 0; pt < KPARTS; ++pt) o += o_s[pt][g][d];
    // every thread carries identical m_run/l_run, select by g without dynamic register indexing
    float l = 0.f, m = 0.f;
#pragma unroll
    for (int gg = 0; gg < GMAX; ++gg)
      if (gg == g) {
        l = l_run[gg];
        m = m_run[gg];
      }
    const int hq = h * G + g;
    if (num_splits == 1) {
      out[(long long)b * out_stride + (long long)hq * D + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
    } else {
      const long long base = ((long long)b * Hq + hq) * num_splits + split;
      o_part[base * D + d] = o;
      if (d == 0) {
        ml_part[base * 2] = m;
        ml_part[base * 2 + 1] = l;
      }
    }
  }
}

template <int D>
__global__ void decode_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part, int Hq,
                                    int num_splits, __nv_bfloat16* __restrict__ out, long long out_stride) {
  const int b = blockIdx.x, hq = blockIdx.y, d = threadIdx.x;
  const long long base = ((long long)b * Hq + hq) * num_splits;
  float m = -INFINITY;
  for (int s = 0; s < num_splits; ++s) m = fmaxf(m, ml_part[(base + s) * 2]);
  float l = 0.f, o = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float ms = ml_part[(base + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : __expf(ms - m);
    l += ml_part[(base + s) * 2 + 1] * w;
    o += o_part[(base + s) * D + d] * w;
  }
  out[(long long)b * out_stride + (long long)hq * D + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
}

// k, v: [T, Hk, D] (token stride given); slot = block * block_size + offset, slot < 0 skips the token.
__global__ void kv_write_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                long long k_stride, long long v_stride, const long long* __restrict__ slots,
                                __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc, long long T, int Hk,
                                int D, int block_size) {
  pdl_trigger();
  pdl_wait();
  const int vec_per_tok = Hk * D / 8;
  const long long total = T * vec_per_tok;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / vec_per_tok;
    const int r = idx % vec_per_tok;
    const long long slot = slots[t];
    if (slot < 0) continue;
    const int h = (r * 8) / D, d = (r * 8) % D;
    const long long blk = slot / block_size, off = slot % block_size;
    const long long dst = ((blk * Hk + h) * block_size + off) * D + d;
    *reinterpret_cast<uint4*>(kc + dst) = *reinterpret_cast<const uint4*>(k + t * k_stride + (long long)h * D + d);
    *reinterpret_cast<uint4*>(vc + dst) = *reinterpret_cast<const uint4*>(v + t * v_stride + (long long)h * D + d);
  }
}

}  // namespace vb

using namespace vb;

extern "C" int vb_decode_num_splits(int B, int Hk, int max_seq_len) {
  const int ctas = B * Hk;
  const int target = 2 * vb_num_sms();
  int s = (target + ctas - 1) / ctas;
  const int chunks = (max_seq_len + CHUNK - 1) / CHUNK;
  if (s > chunks) s = chunks;
  if (s > 16) s = 16;
  if (s < 1) s = 1;
  return s;
}

// Merge of the per-split partial results (head_dim 128), shared with the tensor-core decode kernel.
int vb_decode_merge_128(const float* o_part, const float* ml_part, int B, int Hq, int num_splits, void* out,
                        long long out_stride, cudaStream_t stream) {
  decode_merge_kernel<128><<<dim3(B, Hq), 128, 0, stream>>>(o_part, ml_part, Hq, num_splits, (__nv_bfloat16*)out,
                                                            out_stride);
  return (int)cudaGetLastError();
}

// work: fp32 scratch of B * Hq * num_splits * (D + 2) floats (unused when num_splits == 1).
extern "C" int vb_paged_decode(const void* q, long long q_stride, const void* kc, const void* vc,
                               const int* block_table, int max_blocks, const int* seq_lens, int B, int Hq, int Hk,
                               int D, int block_size, float scale, int num_splits, void* out, long long out_stride,
                               float* work, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (Hq % Hk != 0 || Hq / Hk > GMAX) return -3;
  float* o_part = work;
  float* ml_part = work ? work + (long long)B * Hq * num_splits * D : nullptr;
  dim3 grid(B, Hk, num_splits);
  if (D == 128) {
    paged_decode_kernel<128><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)kc,
                                                       (const __nv_bfloat16*)vc, block_table, max_blocks, seq_lens,
                                                       Hq, Hk, block_size, scale, num_splits, (__nv_bfloat16*)out,
                                                       out_stride, o_part, ml_part);
    if (num_splits > 1)
      decode_merge_kernel<128><<<dim3(B, Hq), 128, 0, stream>>>(o_part, ml_part, Hq, num_splits, (__nv_bfloat16*)out,
                                                                out_stride);
  } else if (D == 64) {
    paged_decode_kernel<64><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)kc,
                                                      (const __nv_bfloat16*)vc, block_table, max_blocks, seq_lens, Hq,
                                                      Hk, block_size, scale, num_splits, (__nv_bfloat16*)out,
                                                      out_stride, o_part, ml_part);
    if (num_splits > 1)
      decode_merge_kernel<64><<<dim3(B, Hq), 64, 0, stream>>>(o_part, ml_part, Hq, num_splits, (__nv_bfloat16*)out,
                                                              out_stride);
  } else {
    return -3;
  }
  vb_count_launch(num_splits > 1 ? 2 : 1);
  return (int)cudaGetLastError();
}

extern "C" int vb_kv_cache_write(const void* k, const void* v, long long k_stride, long long v_stride,
                                 const long long* slots, void* kc, void* vc, long long T, int Hk, int D,
                                 int block_size, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D & 7) return -3;
  long long g = (T * (Hk * D / 8) + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  cudaError_t e = vb_launch_pdl(kv_write_kernel, dim3((unsigned)g), dim3(256), 0, stream, 1, (const __nv_bfloat16*)k,
                                (const __nv_bfloat16*)v, k_stride, v_stride, slots, (__nv_bfloat16*)kc,
                                (__nv_bfloat16*)vc, T, Hk, D, block_size);
  vb_count_launch();
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
