// Block-scaled fp8 (e4m3) GEMM and the quantisation kernels that feed it.
//
// Scaling scheme of the reference's fp8 rollout path (verl/utils/kernel/fp8_kernel.py:53-106, 312;
// verl/utils/vllm/vllm_fp8_utils.py:182-431): weights carry one fp32 scale per 128 x 128 block, activations one per
// (row, 128 columns); scale = absmax / 448, optionally rounded up to a power of two (UE8M0-representable).
//
//   vb_fp8_quant_weight   W [N, K] bf16 -> Wq [N, K] e4m3 + sw [ceil(N/128), ceil(K/128)] fp32
//   vb_fp8_quant_act      X [M, K] bf16 -> Xq [M, K] e4m3 + sx [M, ceil(K/128)] fp32
//   vb_fp8_gemm_blockscale  C[M, N] (bf16) = sum over 128-wide k blocks of (Xq_kb . Wq_kb^T) * sx[m, kb] * sw[nb, kb]
//
// GEMM: one CTA per 128 x 128 output tile (persistent over tiles). Per k block the tensor core computes the
// unscaled partial product with tcgen05.mma kind::f8f6f4 (4 MMAs of K = 32) into one of two TMEM buffers; the four
// epilogue warps read the partial, multiply by the two scales and accumulate in registers while the MMA of the
// next k block runs into the other buffer ("promotion" of every 128-deep partial sum to fp32 outside the tensor
// core, which is what block scaling with plain fp32 scales requires).
#include "common.cuh"
#include "host_utils.h"

#include <cuda_fp8.h>

namespace vb {

constexpr float FP8_MAX = 448.f;

__device__ __forceinline__ float scale_of(float amax, int pow2) {
  float s = fmaxf(amax, 1e-10f) / FP8_MAX;
  if (pow2) {
    // smallest power of two >= s, from the exponent bits (log2f under fast-math is not exact at powers of two)
    int e;
    const float m = frexpf(s, &e);  // s = m * 2^e, m in [0.5, 1)
    s = ldexpf(1.f, m == 0.5f ? e - 1 : e);
  }
  return s;
}

// one block (256 threads) per 128 x 128 tile of W
__global__ void fp8_quant_weight_kernel(const __nv_bfloat16* __restrict__ w, long long ldw, int N, int K,
                                        __nv_fp8_storage_t* __restrict__ q, long long ldq, float* __restrict__ scales,
                                        int pow2) {
  const int nb = blockIdx.y, kb = blockIdx.x;
  const int n0 = nb * 128, k0 = kb * 128;
  __shared__ float red[8];
  __shared__ float s_scale;
  float amax = 0.f;
  for (int i = threadIdx.x; i < 128 * 128; i += blockDim.x) {
    const int r = n0 + i / 128, c = k0 + i % 128;
    if (r < N && c < K) amax = fmaxf(amax, fabsf(__bfloat162float(w[(long long)r * ldw + c])));
  }
  amax = warp_reduce_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) m = fmaxf(m, red[i]);
    s_scale = scale_of(m, pow2);
    scales[(long long)nb * gridDim.x + kb] = s_scale;
  }
  __syncthreads();
  const float inv = 1.f / s_scale;
  for (int i = threadIdx.x; i < 128 * 128; i += blockDim.x) {
    const int r = n0 + i / 128, c = k0 + i % 128;
    if (r < N && c < K)
      q[(long long)r * ldq + c] = __nv_cvt_float_to_fp8(__bfloat162float(w[(long long)r * ldw + c]) * inv, __NV_SATFINITE, __NV_E4M3);
  }
}

// one warp per (row, 128-column block)
__global__ void fp8_quant_act_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, long long M, int K,
                                     __nv_fp8_storage_t* __restrict__ q, long long ldq, float* __restrict__ scales, int pow2) {
  const int nkb = (K + 127) / 128;
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= M * nkb) return;
  const long long row = unit / nkb;
  const int kb = (int)(unit % nkb), lane = threadIdx.x & 31;
  const int c0 = kb * 128 + lane * 4;
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = (c0 + i < K) ? __bfloat162float(x[row * ldx + c0 + i]) : 0.f;
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = warp_reduce_max(amax);
  const float s = scale_of(amax, pow2), inv = 1.f / s;
  if (lane == 0) scales[row * nkb + kb] = s;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (c0 + i < K) q[row * ldq + c0 + i] = __nv_cvt_float_to_fp8(v[i] * inv, __NV_SATFINITE, __NV_E4M3);
}

// ------------------------------------------------------------------------------------------------ GEMM
constexpr int F8_BM = 128, F8_BN = 128, F8_BK = 128;       // BK in elements = 128 bytes = one swizzle span
constexpr int F8_STAGES = 6;
constexpr int F8_TILE = 128 * 128;                          // 16 KB per operand tile
constexpr int F8_STAGE = 2 * F8_TILE;
constexpr int F8_BAR_OFF = F8_STAGES * F8_STAGE;
constexpr int F8_SMEM = F8_BAR_OFF + (2 * F8_STAGES + 4) * 8 + 16 + 1024;
constexpr int F8_THREADS = 192;

struct F8Params {
  int M, N, K;
  __nv_bfloat16* C;
  long long ldc;
  const float* sx;  // [M, nkb]
  const float* sw;  // [ceil(N/128), nkb]
  const __nv_bfloat16* bias;
  int* status;
};

__global__ void __launch_bounds__(F8_THREADS, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const F8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + F8_BAR_OFF);
  uint64_t* empty = full + F8_STAGES;
  uint64_t* pfull = empty + F8_STAGES;   // [2] partial of a k block is in TMEM buffer i
  uint64_t* pempty = pfull + 2;          // [2] the epilogue warps have read buffer i
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + F8_BM - 1) / F8_BM, num_n = (p.N + F8_BN - 1) / F8_BN;
  const int num_kb = (p.K + F8_BK - 1) / F8_BK;
  const int num_tiles = num_m * num_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < F8_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&pfull[i], 1);
      mbar_init(&pempty[i], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
        const int mb = t % num_m, nb = t / num_m;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (*abort_flag || !mbar_wait(&empty[s], phase ^ 1)) {
            report_error(p.status, ERR_WAIT_EMPTY, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full[s], F8_STAGE);
          tma_load_2d(smem + s * F8_STAGE, &tmA, &full[s], kb * F8_BK, mb * F8_BM);
          tma_load_2d(smem + s * F8_STAGE + F8_TILE, &tmB, &full[s], kb * F8_BK, nb * F8_BN);
          if (++s == F8_STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // kind::f8f6f4: formats 0 = e4m3 for both operands, K-major, fp32 accumulate, M = N = 128, K = 32 per MMA
      constexpr uint32_t idesc = umma_idesc(0, 0, 0, 0, F8_BM, F8_BN);
      int s = 0;
      uint32_t phase = 0;
      long long it = 0;  // running k-block counter: TMEM buffer = it & 1
      bool ok = true;
      for (int t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int buf = (int)(it & 1);
          if (*abort_flag || !mbar_wait(&pempty[buf], (uint32_t)((it >> 1) & 1) ^ 1) || !mbar_wait(&full[s], phase)) {
            report_error(p.status, ERR_WAIT_FULL, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * F8_STAGE), b_addr = a_addr + F8_TILE;
#pragma unroll
          for (int k = 0; k < F8_BK / 32; ++k)
            tc_mma_f8(tmem_base + buf * F8_BN, umma_smem_desc(a_addr + k * 32, 16, 1024), umma_smem_desc(b_addr + k * 32, 16, 1024),
                      idesc, k != 0);
          tc_commit(&empty[s]);
          tc_commit(&pfull[buf]);
          if (++s == F8_STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else {
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_base = ((uint32_t)(quad * 32)) << 16;
    long long it = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
      const int mb = t % num_m, nb = t / num_m;
      const int row = mb * F8_BM + row_in_tile;
      const bool row_ok = row < p.M;
      float acc[F8_BN];
#pragma unroll
      for (int i = 0; i < F8_BN; ++i) acc[i] = 0.f;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int buf = (int)(it & 1);
        if (*abort_flag || !mbar_wait(&pfull[buf], (uint32_t)((it >> 1) & 1))) {
          report_error(p.status, ERR_WAIT_TMEM_FULL, kb);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const float sc = (row_ok ? p.sx[(long long)row * num_kb + kb] : 0.f) * p.sw[(long long)nb * num_kb + kb];
#pragma unroll
        for (int c = 0; c < F8_BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + lane_base + buf * F8_BN + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) acc[c * 32 + e] = fmaf(__uint_as_float(v[e]), sc, acc[c * 32 + e]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pempty[buf]);
      }
      if (ok && row_ok) {
        __nv_bfloat16* dst = p.C + (long long)row * p.ldc + nb * F8_BN;
        const int ncol = min(F8_BN, p.N - nb * F8_BN);
        if (p.bias != nullptr) {
#pragma unroll
          for (int i = 0; i < F8_BN; ++i)
            if (i < ncol) acc[i] += __bfloat162float(p.bias[nb * F8_BN + i]);
        }
        if (ncol == F8_BN && (p.ldc & 7) == 0) {
#pragma unroll
          for (int i = 0; i < F8_BN / 8; ++i) {
            uint4 w;
            w.x = pack_bf16x2(acc[8 * i], acc[8 * i + 1]);
            w.y = pack_bf16x2(acc[8 * i + 2], acc[8 * i + 3]);
            w.z = pack_bf16x2(acc[8 * i + 4], acc[8 * i + 5]);
            w.w = pack_bf16x2(acc[8 * i + 6], acc[8 * i + 7]);
            reinterpret_cast<uint4*>(dst)[i] = w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < F8_BN; ++i)
            if (i < ncol) dst[i] = __float2bfloat16(acc[i]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

}  // namespace vb

using namespace vb;

// W [N, K] bf16 (row stride ldw) -> q [N, K] e4m3 (row stride ldq, a multiple of 16) + scales [ceil(N/128), ceil(K/128)].
extern "C" int vb_fp8_quant_weight(const void* w, long long ldw, int N, int K, void* q, long long ldq, float* scales, int pow2,
                                   cudaStream_t stream) {
  if (N <= 0 || K <= 0) return 0;
  dim3 grid((K + 127) / 128, (N + 127) / 128);
  fp8_quant_weight_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(w), ldw, N, K,
                                                    reinterpret_cast<__nv_fp8_storage_t*>(q), ldq, scales, pow2);
  vb_count_launch();
  return (int)cudaGetLastError();
}

// X [M, K] bf16 -> q [M, K] e4m3 + scales [M, ceil(K/128)].
extern "C" int vb_fp8_quant_act(const void* x, long long ldx, long long M, int K, void* q, long long ldq, float* scales,
                                int pow2, cudaStream_t stream) {
  if (M <= 0 || K <= 0) return 0;
  const long long units = M * ((K + 127) / 128);
  fp8_quant_act_kernel<<<(unsigned)((units + 7) / 8), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx, M, K,
                                                                       reinterpret_cast<__nv_fp8_storage_t*>(q), ldq, scales, pow2);
  vb_count_launch();
  return (int)cudaGetLastError();
}

// C [M, N] bf16 = dequantised Xq . Wq^T (+ bias). Xq [M, K], Wq [N, K] e4m3 with row strides (bytes = elements)
// that are multiples of 16; sx [M, ceil(K/128)], sw [ceil(N/128), ceil(K/128)] fp32.
extern "C" int vb_fp8_gemm_blockscale(const void* xq, const void* wq, const float* sx, const float* sw, void* C,
                                      const void* bias, int M, int N, int K, long long ldx, long long ldw, long long ldc,
                                      int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((ldx & 15) || (ldw & 15)) return -3;
  CUtensorMap tmA, tmB;
  int rc = vb_make_tmap_2d(&tmA, xq, 1, (uint64_t)K, (uint64_t)M, (uint64_t)ldx, F8_BK, F8_BM);
  if (rc) return rc;
  rc = vb_make_tmap_2d(&tmB, wq, 1, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, F8_BK, F8_BN);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    VB_CUDA_CHECK(cudaFuncSetAttribute(fp8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM));
    attr_set = true;
  }
  F8Params p{};
  p.M = M; p.N = N; p.K = K;
  p.C = reinterpret_cast<__nv_bfloat16*>(C); p.ldc = ldc;
  p.sx = sx; p.sw = sw; p.bias = reinterpret_cast<const __nv_bfloat16*>(bias); p.status = status;
  const int tiles = ((M + F8_BM - 1) / F8_BM) * ((N + F8_BN - 1) / F8_BN);
  const int grid = tiles < vb_num_sms() ? tiles : vb_num_sms();
  fp8_gemm_kernel<<<grid, F8_THREADS, F8_SMEM, stream>>>(tmA, tmB, p);
  vb_count_launch();
  return (int)cudaGetLastError();
}
