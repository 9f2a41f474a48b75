// Variable-length causal GQA attention, backward, on tcgen05 (head_dim 128). Three kernels:
//
//   flash_bwd_delta   delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]                       (one warp per row)
//   flash_bwd_dq      one CTA per (sequence, query head, 128 queries), loop over key chunks j:
//                         S  = Q K_j^T,  dP = dO V_j^T                (tcgen05, accumulators in TMEM)
//                         dS = exp(S * scale - lse) * (dP - delta) * scale   (thread = query row) -> shared memory
//                         dQ += dS K_j                                (K_j tile reused as MN-major operand)
//   flash_bwd_dkv     one CTA per (sequence, KV head, 128 keys), loop over the query heads of the group and
//                     over query blocks i of 64 rows:
//                         S^T = K Q_i^T,  dP^T = V dO_i^T             (thread = key row)
//                         P^T, dS^T -> shared memory;  dV += P^T dO_i,  dK += dS^T Q_i
//                     dK / dV accumulate in TMEM over the whole loop: no atomics, deterministic.
//
// The probabilities are recomputed from the saved log-sum-exp, as in the forward pass nothing of size [T, T]
// ever exists in memory. All waits are bounded (status word + clean teardown).
#include "common.cuh"
#include "host_utils.h"

namespace vb {

constexpr int FB_D = 128;
constexpr int FB_TILE = 128 * FB_D * 2;  // 32 KB: 128 rows x 128 dims bf16, two 64-dim halves of 16 KB
constexpr int FB_THREADS = 192;

struct FbParams {
  const int* cu_seqlens;
  const float* lse;     // [Hq, T]
  const float* delta;   // [Hq, T]
  __nv_bfloat16* dq;    // [T, Hq, 128]
  __nv_bfloat16* dk;    // [T, Hk, 128]
  __nv_bfloat16* dv;
  long long dq_stride, dkv_stride;
  long long T;
  int Hq, Hk;
  float scale;
  int causal;
  int max_blocks;
  int* status;
};

__device__ __forceinline__ uint32_t fb_sw128(int r, int k) {
  // element (row r, col k) of a K-major bf16 operand with 128-byte swizzle stored as 64-column blocks of
  // (rows * 128) bytes; rows is 128 here
  return (uint32_t)((k >> 6) * 16384 + (r >> 3) * 1024 + (r & 7) * 128 + ((((k & 63) >> 3) ^ (r & 7)) << 4) + (k & 7) * 2);
}

// ------------------------------------------------------------------------------------------------- delta
__global__ void flash_bwd_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                       long long o_stride, long long do_stride, float* __restrict__ delta, long long T,
                                       int Hq) {
  const long long row = (long long)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
  if (row >= T * Hq) return;
  const long long t = row / Hq;
  const int h = (int)(row % Hq), lane = threadIdx.x & 31;
  const uint2 a = *reinterpret_cast<const uint2*>(o + t * o_stride + (long long)h * FB_D + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(dout + t * do_stride + (long long)h * FB_D + lane * 4);
  const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float2 x = __bfloat1622float2(a2[i]), y = __bfloat1622float2(b2[i]);
    s += x.x * y.x + x.y * y.y;
  }
  s = warp_reduce_sum(s);
  if (lane == 0) delta[(long long)h * T + t] = s;
}

// ------------------------------------------------------------------------------------------------- dQ
// Shared memory: Q, dO (resident), dS (one buffer), two K slots and two V slots. K_j has to outlive V_j (it is read
// again by dQ += dS_j K_j), so the two streams have their own rings: a common ring would make the load of V_{j+1}
// wait for a slot that only dQ_j releases, while dQ_j waits for chunk j+1 to be issued.
constexpr int DQ_SLOTS = 2;
constexpr int DQ_Q_OFF = 0, DQ_DO_OFF = FB_TILE, DQ_DS_OFF = 2 * FB_TILE, DQ_K_OFF = 3 * FB_TILE, DQ_V_OFF = 5 * FB_TILE;
constexpr int DQ_BAR_OFF = 7 * FB_TILE;
constexpr int DQ_SMEM = DQ_BAR_OFF + 16 * 8 + 16 + 1024;

__global__ void __launch_bounds__(FB_THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const FbParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem + DQ_Q_OFF;
  uint8_t* do_s = smem + DQ_DO_OFF;
  uint8_t* ds_s = smem + DQ_DS_OFF;
  uint8_t* k_ring = smem + DQ_K_OFF;
  uint8_t* v_ring = smem + DQ_V_OFF;
  uint64_t* kfull = reinterpret_cast<uint64_t*>(smem + DQ_BAR_OFF);
  uint64_t* kempty = kfull + DQ_SLOTS;
  uint64_t* vfull = kempty + DQ_SLOTS;
  uint64_t* vempty = vfull + DQ_SLOTS;
  uint64_t* s_full = vempty + DQ_SLOTS;  // S and dP of chunk j are in TMEM
  uint64_t* ds_ready = s_full + 1;       // dS of chunk j is in shared memory, S / dP may be overwritten
  uint64_t* dq_full = ds_ready + 1;
  uint64_t* qdo_full = dq_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(qdo_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z, hq = blockIdx.y;
  const int qblk = p.max_blocks - 1 - (int)blockIdx.x;
  const int seq_start = p.cu_seqlens[b];
  const int seq_len = p.cu_seqlens[b + 1] - seq_start;
  const int r0 = qblk * 128;
  if (r0 >= seq_len) return;
  const int hk = hq / (p.Hq / p.Hk);
  const int kv_chunks = (seq_len + 127) / 128;
  const int n_chunks = p.causal ? min(kv_chunks, qblk + 1) : kv_chunks;

  if (tid == 0) {
    for (int s = 0; s < DQ_SLOTS; ++s) {
      mbar_init(&kfull[s], 1);
      mbar_init(&kempty[s], 1);
      mbar_init(&vfull[s], 1);
      mbar_init(&vempty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(ds_ready, 4);
    mbar_init(dq_full, 1);
    mbar_init(qdo_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DQ = 256;

  if (warp == 4) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmDO);
      mbar_arrive_expect_tx(qdo_full, 2 * FB_TILE);
      tma_load_2d(q_s, &tmQ, qdo_full, hq * FB_D, seq_start + r0);
      tma_load_2d(q_s + 16384, &tmQ, qdo_full, hq * FB_D + 64, seq_start + r0);
      tma_load_2d(do_s, &tmDO, qdo_full, hq * FB_D, seq_start + r0);
      tma_load_2d(do_s + 16384, &tmDO, qdo_full, hq * FB_D + 64, seq_start + r0);
      for (int j = 0; j < n_chunks; ++j) {
        const int s = j % DQ_SLOTS;
        const uint32_t par = ((j / DQ_SLOTS) & 1) ^ 1;
        const int row = seq_start + j * 128;
        if (*abort_flag || !mbar_wait(&kempty[s], par)) {
          report_error(p.status, ERR_WAIT_EMPTY, 2 * j);
          *abort_flag = 1;
          break;
        }
        mbar_arrive_expect_tx(&kfull[s], FB_TILE);
        tma_load_2d(k_ring + s * FB_TILE, &tmK, &kfull[s], hk * FB_D, row);
        tma_load_2d(k_ring + s * FB_TILE + 16384, &tmK, &kfull[s], hk * FB_D + 64, row);
        if (*abort_flag || !mbar_wait(&vempty[s], par)) {
          report_error(p.status, ERR_WAIT_EMPTY, 2 * j + 1);
          *abort_flag = 1;
          break;
        }
        mbar_arrive_expect_tx(&vfull[s], FB_TILE);
        tma_load_2d(v_ring + s * FB_TILE, &tmV, &vfull[s], hk * FB_D, row);
        tma_load_2d(v_ring + s * FB_TILE + 16384, &tmV, &vfull[s], hk * FB_D + 64, row);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = umma_idesc(1, 1, 0, 0, 128, 128);  // both operands K-major
      constexpr uint32_t idesc_kn = umma_idesc(1, 1, 0, 1, 128, 128);  // B MN-major
      const uint32_t q_addr = smem_u32(q_s), do_addr = smem_u32(do_s);
      bool ok = !*abort_flag && mbar_wait(qdo_full, 0);
      if (!ok) {
        report_error(p.status, ERR_WAIT_FULL, 9000);
        *abort_flag = 1;
      }
      auto issue_dq = [&](int j) {  // dQ += dS_j . K_j, then K_j's slot is free
        const int s = j % DQ_SLOTS;
        const uint32_t k_addr = smem_u32(k_ring + s * FB_TILE);
        const uint32_t ds_addr = smem_u32(ds_s);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          tc_mma_f16(tmem_base + TM_DQ, umma_smem_desc(ds_addr + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                     umma_smem_desc(k_addr + k * 2048, 16384, 1024), idesc_kn, (j | k) != 0);
        tc_commit(&kempty[s]);
      };
      for (int j = 0; ok && j < n_chunks; ++j) {
        if (j > 0) {
          // S / dP of chunk j-1 have been read and dS_{j-1} is in shared memory: dQ first, so that it is complete
          // (and the dS buffer free again) by the time S / dP of chunk j are
          if (*abort_flag || !mbar_wait(ds_ready, (j - 1) & 1)) {
            report_error(p.status, ERR_WAIT_TMEM_EMPTY, j);
            *abort_flag = 1;
            break;
          }
          tc_fence_after();
          issue_dq(j - 1);
        }
        const int s = j % DQ_SLOTS;
        const uint32_t par = (j / DQ_SLOTS) & 1;
        if (*abort_flag || !mbar_wait(&kfull[s], par) || !mbar_wait(&vfull[s], par)) {
          report_error(p.status, ERR_WAIT_FULL, j);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(k_ring + s * FB_TILE);
        const uint32_t v_addr = smem_u32(v_ring + s * FB_TILE);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          tc_mma_f16(tmem_base + TM_S, umma_smem_desc(q_addr + off, 16, 1024), umma_smem_desc(k_addr + off, 16, 1024),
                     idesc_kk, k != 0);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          tc_mma_f16(tmem_base + TM_DP, umma_smem_desc(do_addr + off, 16, 1024), umma_smem_desc(v_addr + off, 16, 1024),
                     idesc_kk, k != 0);
        }
        tc_commit(s_full);
        tc_commit(&vempty[s]);
      }
      if (ok && n_chunks > 0 && !*abort_flag) {
        const int j = n_chunks - 1;
        if (mbar_wait(ds_ready, j & 1)) {
          tc_fence_after();
          issue_dq(j);
          tc_commit(dq_full);
        } else {
          report_error(p.status, ERR_WAIT_TMEM_EMPTY, 7000);
          *abort_flag = 1;
        }
      }
    }
  } else {
    const int r = tid;
    const int qpos = r0 + r;
    const bool row_ok = qpos < seq_len;
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    const float lse = row_ok ? p.lse[(long long)hq * p.T + seq_start + qpos] : 0.f;
    const float delta = row_ok ? p.delta[(long long)hq * p.T + seq_start + qpos] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_chunks; ++j) {
      if (*abort_flag || !mbar_wait(s_full, j & 1)) {
        report_error(p.status, ERR_WAIT_TMEM_FULL, j);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      const int c0 = j * 128;
      int lim = seq_len - c0;
      if (p.causal) lim = min(lim, qpos - c0 + 1);
      lim = row_ok ? max(min(lim, 128), 0) : 0;
      uint8_t* dsbuf = ds_s;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(tmem_base + lane_base + TM_S + c * 32, sv);
        tmem_ld_32x32(tmem_base + lane_base + TM_DP + c * 32, dv);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float d0 = 0.f, d1 = 0.f;
          if (c * 32 + e < lim) d0 = __expf(__uint_as_float(sv[e]) * p.scale - lse) * (__uint_as_float(dv[e]) - delta) * p.scale;
          if (c * 32 + e + 1 < lim)
            d1 = __expf(__uint_as_float(sv[e + 1]) * p.scale - lse) * (__uint_as_float(dv[e + 1]) - delta) * p.scale;
          packed[e >> 1] = pack_bf16x2(d0, d1);
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4)
          *reinterpret_cast<uint4*>(dsbuf + fb_sw128(r, c * 32 + q4 * 8)) =
              make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
    }
    if (ok && (*abort_flag || !mbar_wait(dq_full, 0))) {
      report_error(p.status, ERR_WAIT_TMEM_FULL, 8000);
      *abort_flag = 1;
      ok = false;
    }
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dst = p.dq + (long long)(seq_start + qpos) * p.dq_stride + (long long)hq * FB_D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + lane_base + TM_DQ + c * 32, v);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(v[8 * i]), __uint_as_float(v[8 * i + 1]));
            w.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3]));
            w.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5]));
            w.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7]));
            reinterpret_cast<uint4*>(dst + c * 32)[i] = w;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------- dK / dV
constexpr int KV_QROWS = 64;                       // query rows per iteration
constexpr int KV_QTILE = KV_QROWS * FB_D * 2;      // 16 KB: two 64-dim halves of 8 KB
constexpr int KV_STAGE = 2 * KV_QTILE;             // Q_i and dO_i
constexpr int KV_PT = 128 * KV_QROWS * 2;          // 16 KB: P^T or dS^T, [128 keys x 64 queries]
constexpr int KV_K_OFF = 0, KV_V_OFF = FB_TILE, KV_RING_OFF = 2 * FB_TILE, KV_P_OFF = KV_RING_OFF + 2 * KV_STAGE;
constexpr int KV_LD_OFF = KV_P_OFF + 4 * KV_PT;    // lse / delta of the current query rows: [2 buffers][2][64] floats
constexpr int KV_BAR_OFF = KV_LD_OFF + 2 * 2 * KV_QROWS * 4;
constexpr int KV_SMEM = KV_BAR_OFF + 16 * 8 + 16 + 1024;

__global__ void __launch_bounds__(FB_THREADS, 1)
flash_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const FbParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_s = smem + KV_K_OFF;
  uint8_t* v_s = smem + KV_V_OFF;
  uint8_t* ring = smem + KV_RING_OFF;
  uint8_t* pt_s = smem + KV_P_OFF;  // [buffer][P^T | dS^T]
  float* ld_s = reinterpret_cast<float*>(smem + KV_LD_OFF);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + KV_BAR_OFF);
  uint64_t* empty = full + 2;
  uint64_t* s_full = empty + 2;
  uint64_t* p_ready = s_full + 2;
  uint64_t* kv_full = p_ready + 2;
  uint64_t* acc_full = kv_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z, hk = blockIdx.y, kblk = blockIdx.x;
  const int seq_start = p.cu_seqlens[b];
  const int seq_len = p.cu_seqlens[b + 1] - seq_start;
  const int c0 = kblk * 128;
  if (c0 >= seq_len) return;
  const int G = p.Hq / p.Hk;
  const int n_q64 = (seq_len + KV_QROWS - 1) / KV_QROWS;
  const int i_first = p.causal ? c0 / KV_QROWS : 0;  // earlier query rows never see these keys
  const int per_head = n_q64 - i_first;
  const int n_iter = G * per_head;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);
    }
    mbar_init(kv_full, 1);
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t TM_ST = 0, TM_DPT = 128, TM_DV = 256, TM_DK = 384;  // S^T / dP^T: two 64-column buffers each

  if (warp == 4) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmDO);
      mbar_arrive_expect_tx(kv_full, 2 * FB_TILE);
      tma_load_2d(k_s, &tmK, kv_full, hk * FB_D, seq_start + c0);
      tma_load_2d(k_s + 16384, &tmK, kv_full, hk * FB_D + 64, seq_start + c0);
      tma_load_2d(v_s, &tmV, kv_full, hk * FB_D, seq_start + c0);
      tma_load_2d(v_s + 16384, &tmV, kv_full, hk * FB_D + 64, seq_start + c0);
      for (int t = 0; t < n_iter; ++t) {
        const int s = t & 1;
        if (*abort_flag || !mbar_wait(&empty[s], ((t >> 1) & 1) ^ 1)) {
          report_error(p.status, ERR_WAIT_EMPTY, t);
          *abort_flag = 1;
          break;
        }
        const int hq = hk * G + t / per_head;
        const int row = seq_start + (i_first + t % per_head) * KV_QROWS;
        uint8_t* dst = ring + s * KV_STAGE;
        mbar_arrive_expect_tx(&full[s], KV_STAGE);
        tma_load_2d(dst, &tmQ, &full[s], hq * FB_D, row);
        tma_load_2d(dst + 8192, &tmQ, &full[s], hq * FB_D + 64, row);
        tma_load_2d(dst + KV_QTILE, &tmDO, &full[s], hq * FB_D, row);
        tma_load_2d(dst + KV_QTILE + 8192, &tmDO, &full[s], hq * FB_D + 64, row);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc_st = umma_idesc(1, 1, 0, 0, 128, KV_QROWS);  // S^T / dP^T: both operands K-major
      constexpr uint32_t idesc_acc = umma_idesc(1, 1, 0, 1, 128, FB_D);     // dV / dK: B (dO_i, Q_i) MN-major
      const uint32_t k_addr = smem_u32(k_s), v_addr = smem_u32(v_s);
      bool ok = !*abort_flag && mbar_wait(kv_full, 0);
      if (!ok) {
        report_error(p.status, ERR_WAIT_FULL, 9000);
        *abort_flag = 1;
      }
      auto issue_st = [&](int t) -> bool {
        const int s = t & 1;
        if (*abort_flag || !mbar_wait(&full[s], (t >> 1) & 1)) {
          report_error(p.status, ERR_WAIT_FULL, t);
          *abort_flag = 1;
          return false;
        }
        tc_fence_after();
        const uint32_t q_addr = smem_u32(ring + s * KV_STAGE), do_addr = q_addr + KV_QTILE;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          tc_mma_f16(tmem_base + TM_ST + s * KV_QROWS, umma_smem_desc(k_addr + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                     umma_smem_desc(q_addr + (k >> 2) * 8192 + (k & 3) * 32, 16, 1024), idesc_st, k != 0);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          tc_mma_f16(tmem_base + TM_DPT + s * KV_QROWS, umma_smem_desc(v_addr + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                     umma_smem_desc(do_addr + (k >> 2) * 8192 + (k & 3) * 32, 16, 1024), idesc_st, k != 0);
        tc_commit(&s_full[s]);
        return true;
      };
      if (ok && n_iter > 0) ok = issue_st(0);
      for (int t = 0; ok && t < n_iter; ++t) {
        if (t + 1 < n_iter) ok = issue_st(t + 1);
        if (!ok) break;
        const int s = t & 1;
        if (*abort_flag || !mbar_wait(&p_ready[s], (t >> 1) & 1)) {
          report_error(p.status, ERR_WAIT_TMEM_EMPTY, t);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t q_addr = smem_u32(ring + s * KV_STAGE), do_addr = q_addr + KV_QTILE;
        const uint32_t pt_addr = smem_u32(pt_s + s * 2 * KV_PT), dst_addr = pt_addr + KV_PT;
#pragma unroll
        for (int k = 0; k < KV_QROWS / 16; ++k) {
          // A: [128 keys x 64 queries] K-major, one 64-column block; B: [64 query rows, 128 dims] MN-major
          tc_mma_f16(tmem_base + TM_DV, umma_smem_desc(pt_addr + k * 32, 16, 1024), umma_smem_desc(do_addr + k * 2048, 8192, 1024),
                     idesc_acc, (t | k) != 0);
        }
#pragma unroll
        for (int k = 0; k < KV_QROWS / 16; ++k)
          tc_mma_f16(tmem_base + TM_DK, umma_smem_desc(dst_addr + k * 32, 16, 1024), umma_smem_desc(q_addr + k * 2048, 8192, 1024),
                     idesc_acc, (t | k) != 0);
        tc_commit(&empty[s]);
      }
      if (ok) tc_commit(acc_full);
    }
  } else {
    const int r = tid;               // key row
    const int kpos = c0 + r;
    const bool key_ok = kpos < seq_len;
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    bool ok = true;
    for (int t = 0; t < n_iter; ++t) {
      const int s = t & 1;
      const int hq = hk * G + t / per_head;
      const int q0 = (i_first + t % per_head) * KV_QROWS;
      // lse / delta of the 64 query rows of this iteration (buffer s: the previous use was two iterations ago and
      // every thread has passed a barrier since)
      float* ld = ld_s + s * 2 * KV_QROWS;
      if (tid < 2 * KV_QROWS) {
        const int q = q0 + (tid & (KV_QROWS - 1));
        const float* src = (tid < KV_QROWS) ? p.lse : p.delta;
        ld[tid] = (q < seq_len) ? src[(long long)hq * p.T + seq_start + q] : 0.f;
      }
      {
        // barrier for the staged values that also and-reduces `ok`: a wait that ran out ends the loop for all 128
        // threads in the same iteration (nobody is left alone at a barrier)
        uint32_t all_ok;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.red.and.pred p, 1, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(all_ok)
            : "r"((uint32_t)(ok ? 1 : 0))
            : "memory");
        if (!all_ok) {
          ok = false;
          break;
        }
      }
      if (*abort_flag || !mbar_wait(&s_full[s], (t >> 1) & 1)) {
        report_error(p.status, ERR_WAIT_TMEM_FULL, t);
        *abort_flag = 1;
        ok = false;
      }
      uint8_t* pbuf = pt_s + s * 2 * KV_PT;
      uint8_t* dsbuf = pbuf + KV_PT;
      if (ok) {
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < KV_QROWS / 32; ++c) {
          uint32_t sv[32], dv[32];
          tmem_ld_32x32(tmem_base + lane_base + TM_ST + s * KV_QROWS + c * 32, sv);
          tmem_ld_32x32(tmem_base + lane_base + TM_DPT + s * KV_QROWS + c * 32, dv);
          tmem_ld_wait();
          uint32_t pp[16], dd[16];
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float pv[2], dsv[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int col = c * 32 + e + h;
              const int q = q0 + col;
              const bool vis = key_ok && q < seq_len && (!p.causal || kpos <= q);
              const float pr = vis ? __expf(__uint_as_float(sv[e + h]) * p.scale - ld[col]) : 0.f;
              pv[h] = pr;
              dsv[h] = pr * (__uint_as_float(dv[e + h]) - ld[KV_QROWS + col]) * p.scale;
            }
            pp[e >> 1] = pack_bf16x2(pv[0], pv[1]);
            dd[e >> 1] = pack_bf16x2(dsv[0], dsv[1]);
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const uint32_t off = fb_sw128(r, c * 32 + q4 * 8);
            *reinterpret_cast<uint4*>(pbuf + off) = make_uint4(pp[4 * q4], pp[4 * q4 + 1], pp[4 * q4 + 2], pp[4 * q4 + 3]);
            *reinterpret_cast<uint4*>(dsbuf + off) = make_uint4(dd[4 * q4], dd[4 * q4 + 1], dd[4 * q4 + 2], dd[4 * q4 + 3]);
          }
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[s]);
    }
    if (ok && (*abort_flag || !mbar_wait(acc_full, 0))) {
      report_error(p.status, ERR_WAIT_TMEM_FULL, 8000);
      *abort_flag = 1;
      ok = false;
    }
    if (ok) {
      tc_fence_after();
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* base = which == 0 ? p.dv : p.dk;
        __nv_bfloat16* dst = base + (long long)(seq_start + kpos) * p.dkv_stride + (long long)hk * FB_D;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + lane_base + (which == 0 ? TM_DV : TM_DK) + c * 32, v);
          tmem_ld_wait();
          if (key_ok) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(v[8 * i]), __uint_as_float(v[8 * i + 1]));
              w.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3]));
              w.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5]));
              w.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7]));
              reinterpret_cast<uint4*>(dst + c * 32)[i] = w;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace vb

using namespace vb;

static int fb_tmap(CUtensorMap* tm, const void* ptr, int H, long long T, long long stride, int rows) {
  return vb_make_tmap_2d(tm, ptr, 2, (uint64_t)H * FB_D, (uint64_t)T, (uint64_t)stride * 2, 64, rows);
}

// delta[h, t] = sum_d dO * O; o / dout [T, Hq, 128] bf16 with token strides.
extern "C" int vb_flash_bwd_delta(const void* o, const void* dout, long long o_stride, long long do_stride, float* delta,
                                  long long T, int Hq, cudaStream_t stream) {
  if (T <= 0) return 0;
  const long long rows = T * Hq;
  flash_bwd_delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(o), reinterpret_cast<const __nv_bfloat16*>(dout), o_stride, do_stride, delta, T, Hq);
  vb_count_launch();
  return (int)cudaGetLastError();
}

extern "C" int vb_flash_bwd_dq(const void* q, const void* k, const void* v, const void* dout, long long q_stride,
                               long long k_stride, long long v_stride, long long do_stride, const int* cu_seqlens, int B,
                               long long T, int max_seqlen, int Hq, int Hk, float scale, int causal, const float* lse,
                               const float* delta, void* dq, long long dq_stride, int* status, cudaStream_t stream) {
  if (B <= 0 || T <= 0 || max_seqlen <= 0) return 0;
  if (Hk <= 0 || Hq % Hk != 0 || ((q_stride | k_stride | v_stride | do_stride | dq_stride) & 7)) return -3;
  CUtensorMap tmQ, tmK, tmV, tmDO;
  int rc;
  if ((rc = fb_tmap(&tmQ, q, Hq, T, q_stride, 128))) return rc;
  if ((rc = fb_tmap(&tmK, k, Hk, T, k_stride, 128))) return rc;
  if ((rc = fb_tmap(&tmV, v, Hk, T, v_stride, 128))) return rc;
  if ((rc = fb_tmap(&tmDO, dout, Hq, T, do_stride, 128))) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    VB_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM));
    attr_set = true;
  }
  FbParams p{};
  p.cu_seqlens = cu_seqlens; p.lse = lse; p.delta = delta;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq); p.dq_stride = dq_stride;
  p.T = T; p.Hq = Hq; p.Hk = Hk; p.scale = scale; p.causal = causal;
  p.max_blocks = (max_seqlen + 127) / 128;
  p.status = status;
  flash_bwd_dq_kernel<<<dim3(p.max_blocks, Hq, B), FB_THREADS, DQ_SMEM, stream>>>(tmQ, tmK, tmV, tmDO, p);
  vb_count_launch();
  return (int)cudaGetLastError();
}

// dK, dV [T, Hk, 128] bf16 (token stride dkv_stride): every (sequence, KV head, 128-key block) is owned by one CTA.
extern "C" int vb_flash_bwd_dkv(const void* q, const void* k, const void* v, const void* dout, long long q_stride,
                                long long k_stride, long long v_stride, long long do_stride, const int* cu_seqlens, int B,
                                long long T, int max_seqlen, int Hq, int Hk, float scale, int causal, const float* lse,
                                const float* delta, void* dk, void* dv, long long dkv_stride, int* status,
                                cudaStream_t stream) {
  if (B <= 0 || T <= 0 || max_seqlen <= 0) return 0;
  if (Hk <= 0 || Hq % Hk != 0 || ((q_stride | k_stride | v_stride | do_stride | dkv_stride) & 7)) return -3;
  CUtensorMap tmQ, tmK, tmV, tmDO;
  int rc;
  if ((rc = fb_tmap(&tmQ, q, Hq, T, q_stride, KV_QROWS))) return rc;
  if ((rc = fb_tmap(&tmK, k, Hk, T, k_stride, 128))) return rc;
  if ((rc = fb_tmap(&tmV, v, Hk, T, v_stride, 128))) return rc;
  if ((rc = fb_tmap(&tmDO, dout, Hq, T, do_stride, KV_QROWS))) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    VB_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, KV_SMEM));
    attr_set = true;
  }
  FbParams p{};
  p.cu_seqlens = cu_seqlens; p.lse = lse; p.delta = delta;
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk); p.dv = reinterpret_cast<__nv_bfloat16*>(dv); p.dkv_stride = dkv_stride;
  p.T = T; p.Hq = Hq; p.Hk = Hk; p.scale = scale; p.causal = causal;
  p.max_blocks = (max_seqlen + 127) / 128;
  p.status = status;
  flash_bwd_dkv_kernel<<<dim3(p.max_blocks, Hk, B), FB_THREADS, KV_SMEM, stream>>>(tmQ, tmK, tmV, tmDO, p);
  vb_count_launch();
  return (int)cudaGetLastError();
}
