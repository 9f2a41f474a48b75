// Variable-length causal GQA attention, forward, on tcgen05 (head_dim 128).
//
// One CTA per (sequence, query head, block of 128 queries). Per chunk of 128 keys:
//     S[128 q x 128 keys] = Q . K^T              (tcgen05.mma, both operands K-major, accumulator in TMEM)
//     P = exp(S * scale - rowmax)                (4 softmax warps, one thread per query row: no shuffles)
//     O_c[128 q x 128 dims] = P . V              (P from shared memory, V used as MN-major B operand as stored)
//     O = O * alpha + O_c                        (running output in registers, flash-attention rescale)
// S and O_c are double-buffered in TMEM (4 x 128 columns), P is double-buffered in shared memory, K / V tiles
// arrive through a ring of three 32 KB slots filled by per-CTA TMA loads straight out of the packed [T, H*128]
// tensors (rows of a neighbouring sequence that a tile drags in are masked by position). The softmax of chunk
// c+1 is computed while the tensor core works on P.V of chunk c.
//
// Outputs: O [T, Hq, 128] bf16 and the log-sum-exp per (head, token) in fp32 for the backward pass.
// Every wait is bounded; on expiry the status word is set and the CTA leaves through its teardown.
#include "common.cuh"
#include "host_utils.h"

namespace vb {

constexpr int FA_BM = 128;      // queries per CTA
constexpr int FA_BN = 128;      // keys per chunk
constexpr int FA_D = 128;
constexpr int FA_SLOTS = 3;
constexpr int FA_TILE = FA_BN * FA_D * 2;  // 32 KB
constexpr int FA_THREADS = 192;
constexpr int FA_Q_OFF = 0;
constexpr int FA_P_OFF = FA_TILE;                   // two P buffers
constexpr int FA_RING_OFF = FA_P_OFF + 2 * FA_TILE;
constexpr int FA_BAR_OFF = FA_RING_OFF + FA_SLOTS * FA_TILE;
constexpr int FA_SMEM = FA_BAR_OFF + 16 * 8 + 16 + 1024;

struct FaParams {
  const int* cu_seqlens;  // [B + 1] query side
  const int* cu_k;        // [B + 1] key side, or null when keys and queries are the same tokens
  __nv_bfloat16* out;
  long long out_stride;   // elements between tokens
  float* lse;             // [Hq, T]
  long long T;
  int Hq, Hk;
  float scale;
  int causal;
  int max_qblocks;
  int* status;
};

__device__ __forceinline__ uint32_t fa_sw128(int r, int k) {
  // byte offset of element (row r, col k) in a [128 rows x 128 cols] bf16 K-major operand, 128-byte swizzle,
  // stored as two 64-column blocks of 16 KB
  return (uint32_t)((k >> 6) * 16384 + (r >> 3) * 1024 + (r & 7) * 128 + ((((k & 63) >> 3) ^ (r & 7)) << 4) + (k & 7) * 2);
}

__global__ void __launch_bounds__(FA_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem + FA_Q_OFF;
  uint8_t* p_s = smem + FA_P_OFF;
  uint8_t* ring = smem + FA_RING_OFF;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + FA_BAR_OFF);
  uint64_t* empty = full + FA_SLOTS;
  uint64_t* s_full = empty + FA_SLOTS;
  uint64_t* p_ready = s_full + 2;
  uint64_t* o_full = p_ready + 2;
  uint64_t* q_full = o_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z, hq = blockIdx.y;
  const int qblk = p.max_qblocks - 1 - (int)blockIdx.x;  // long (late) blocks first
  const int seq_start = p.cu_seqlens[b];
  const int seq_len = p.cu_seqlens[b + 1] - seq_start;
  const int r0 = qblk * FA_BM;
  if (r0 >= seq_len) return;  // uniform for the CTA, before any barrier or allocation
  const int hk = hq / (p.Hq / p.Hk);
  // keys may be a longer stream than the queries (prefill on top of a cached prefix): the queries are the last
  // seq_len positions of the seq_len_k keys, i.e. query i sees keys [0, i + koff]
  const int k_start = p.cu_k ? p.cu_k[b] : seq_start;
  const int seq_len_k = p.cu_k ? p.cu_k[b + 1] - k_start : seq_len;
  const int koff = seq_len_k - seq_len;
  const int kv_chunks = (seq_len_k + FA_BN - 1) / FA_BN;
  const int n_chunks = p.causal ? min(kv_chunks, (r0 + FA_BM - 1 + koff) / FA_BN + 1) : kv_chunks;

  if (tid == 0) {
    for (int s = 0; s < FA_SLOTS; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);
      mbar_init(&o_full[i], 1);
    }
    mbar_init(q_full, 1);
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

  if (warp == 4) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_arrive_expect_tx(q_full, FA_TILE);
      tma_load_2d(q_s, &tmQ, q_full, hq * FA_D, seq_start + r0);
      tma_load_2d(q_s + 16384, &tmQ, q_full, hq * FA_D + 64, seq_start + r0);
      for (int t = 0; t < 2 * n_chunks; ++t) {
        const int s = t % FA_SLOTS;
        if (*abort_flag || !mbar_wait(&empty[s], ((t / FA_SLOTS) & 1) ^ 1)) {
          report_error(p.status, ERR_WAIT_EMPTY, t);
          *abort_flag = 1;
          break;
        }
        mbar_arrive_expect_tx(&full[s], FA_TILE);
        uint8_t* dst = ring + s * FA_TILE;
        const CUtensorMap* tm = (t & 1) ? &tmV : &tmK;
        const int row = k_start + (t >> 1) * FA_BN;
        tma_load_2d(dst, tm, &full[s], hk * FA_D, row);
        tma_load_2d(dst + 16384, tm, &full[s], hk * FA_D + 64, row);
      }
    }
  } else if (warp == 5) {
    // -------------------------------- MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(1, 1, 0, 0, FA_BM, FA_BN);  // A = Q, B = K: both K-major
      constexpr uint32_t idesc_pv = umma_idesc(1, 1, 0, 1, FA_BM, FA_D);   // A = P K-major, B = V MN-major
      const uint32_t q_addr = smem_u32(q_s);
      bool ok = !*abort_flag && mbar_wait(q_full, 0);
      if (!ok) {
        report_error(p.status, ERR_WAIT_FULL, 9000);
        *abort_flag = 1;
      }
      auto issue_qk = [&](int c) -> bool {
        const int t = 2 * c, s = t % FA_SLOTS;
        if (*abort_flag || !mbar_wait(&full[s], (t / FA_SLOTS) & 1)) {
          report_error(p.status, ERR_WAIT_FULL, t);
          *abort_flag = 1;
          return false;
        }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(ring + s * FA_TILE);
        const uint32_t d_tmem = tmem_base + (c & 1) * FA_BN;
#pragma unroll
        for (int k = 0; k < FA_D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          tc_mma_f16(d_tmem, umma_smem_desc(q_addr + off, 16, 1024), umma_smem_desc(k_addr + off, 16, 1024), idesc_qk,
                     k != 0);
        }
        tc_commit(&s_full[c & 1]);
        tc_commit(&empty[s]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int c = 0; ok && c < n_chunks; ++c) {
        if (c + 1 < n_chunks) ok = issue_qk(c + 1);
        if (!ok) break;
        const int t = 2 * c + 1, s = t % FA_SLOTS;
        if (*abort_flag || !mbar_wait(&full[s], (t / FA_SLOTS) & 1)) {
          report_error(p.status, ERR_WAIT_FULL, t);
          *abort_flag = 1;
          break;
        }
        if (*abort_flag || !mbar_wait(&p_ready[c & 1], (c >> 1) & 1)) {
          report_error(p.status, ERR_WAIT_TMEM_EMPTY, c);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(ring + s * FA_TILE);
        const uint32_t p_addr = smem_u32(p_s + (c & 1) * FA_TILE);
        const uint32_t d_tmem = tmem_base + 256 + (c & 1) * FA_D;
#pragma unroll
        for (int k = 0; k < FA_BN / 16; ++k) {
          const uint64_t a = umma_smem_desc(p_addr + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
          const uint64_t bv = umma_smem_desc(v_addr + k * 2048, 16384, 1024);
          tc_mma_f16(d_tmem, a, bv, idesc_pv, k != 0);
        }
        tc_commit(&o_full[c & 1]);
        tc_commit(&empty[s]);
      }
    }
  } else {
    // ----------------------- softmax + accumulation (128 threads, thread = query row) -----------------------
    const int r = tid;
    const int qpos = r0 + r;
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    float o_acc[FA_D];
#pragma unroll
    for (int i = 0; i < FA_D; ++i) o_acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    float alpha_cur = 1.f, alpha_nxt = 1.f;
    bool ok = true;

    auto softmax_chunk = [&](int c) -> float {
      const int i = c & 1;
      if (*abort_flag || !mbar_wait(&s_full[i], (c >> 1) & 1)) {
        report_error(p.status, ERR_WAIT_TMEM_FULL, c);
        *abort_flag = 1;
        ok = false;
      }
      const int c0 = c * FA_BN;
      // keys this row may see in the chunk: [0, lim)
      int lim = seq_len_k - c0;
      if (p.causal) lim = min(lim, qpos + koff - c0 + 1);
      lim = max(min(lim, FA_BN), 0);
      const uint32_t s_addr = tmem_base + lane_base + i * FA_BN;
      float cmax = -INFINITY;
      if (ok) {
        tc_fence_after();
#pragma unroll 1
        for (int j = 0; j < FA_BN / 32; ++j) {
          uint32_t v[32];
          tmem_ld_32x32(s_addr + j * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (j * 32 + e < lim) cmax = fmaxf(cmax, __uint_as_float(v[e]));
        }
      }
      cmax *= p.scale;  // scale > 0: max commutes with the scaling
      const float m_new = fmaxf(m_run, cmax);
      // a row without any visible key so far keeps m = -inf; use 0 as the reference to avoid inf - inf
      const float m_ref = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = __expf(m_run - m_ref);
      float lsum = 0.f;
      uint8_t* pbuf = p_s + i * FA_TILE;
      if (ok) {
#pragma unroll 1
        for (int j = 0; j < FA_BN / 32; ++j) {
          uint32_t v[32];
          tmem_ld_32x32(s_addr + j * 32, v);
          tmem_ld_wait();
          uint32_t packed[16];
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float p0 = (j * 32 + e < lim) ? __expf(__uint_as_float(v[e]) * p.scale - m_ref) : 0.f;
            const float p1 = (j * 32 + e + 1 < lim) ? __expf(__uint_as_float(v[e + 1]) * p.scale - m_ref) : 0.f;
            lsum += p0 + p1;
            packed[e >> 1] = pack_bf16x2(p0, p1);
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int k = j * 32 + q4 * 8;
            *reinterpret_cast<uint4*>(pbuf + fa_sw128(r, k)) =
                make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
          }
        }
      }
      m_run = m_new;
      l_run = l_run * alpha + lsum;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[i]);
      return alpha;
    };

    alpha_cur = softmax_chunk(0);
    for (int c = 0; c < n_chunks; ++c) {
      const int i = c & 1;
      if (c + 1 < n_chunks) alpha_nxt = softmax_chunk(c + 1);
      if (ok && (*abort_flag || !mbar_wait(&o_full[i], (c >> 1) & 1))) {
        report_error(p.status, ERR_WAIT_TMEM_FULL, 1000 + c);
        *abort_flag = 1;
        ok = false;
      }
      if (ok) {
        tc_fence_after();
        const uint32_t o_addr = tmem_base + lane_base + 256 + i * FA_D;
#pragma unroll
        for (int j = 0; j < FA_D / 32; ++j) {
          uint32_t v[32];
          tmem_ld_32x32(o_addr + j * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) o_acc[j * 32 + e] = o_acc[j * 32 + e] * alpha_cur + __uint_as_float(v[e]);
        }
      }
      alpha_cur = alpha_nxt;
      if (!ok) break;  // per-thread exit is fine: the softmax threads share no block-level barrier
    }
    if (ok && qpos < seq_len) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = p.out + (long long)(seq_start + qpos) * p.out_stride + (long long)hq * FA_D;
#pragma unroll
      for (int j = 0; j < FA_D / 8; ++j) {
        uint4 w;
        w.x = pack_bf16x2(o_acc[8 * j] * inv, o_acc[8 * j + 1] * inv);
        w.y = pack_bf16x2(o_acc[8 * j + 2] * inv, o_acc[8 * j + 3] * inv);
        w.z = pack_bf16x2(o_acc[8 * j + 4] * inv, o_acc[8 * j + 5] * inv);
        w.w = pack_bf16x2(o_acc[8 * j + 6] * inv, o_acc[8 * j + 7] * inv);
        reinterpret_cast<uint4*>(dst)[j] = w;
      }
      if (p.lse != nullptr) p.lse[(long long)hq * p.T + seq_start + qpos] = (l_run > 0.f) ? m_run + __logf(l_run) : -INFINITY;
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

extern "C" int vb_flash_fwd_supported(int Hq, int Hk, int D) { return (D == FA_D && Hk > 0 && Hq % Hk == 0) ? 1 : 0; }

// q [T, Hq, 128], k / v [Tk, Hk, 128] bf16 with token strides (elements, multiples of 8); cu_seqlens int32 [B + 1] on
// the device; cu_k / Tk describe the key stream when it differs from the query stream (null / 0 otherwise; with
// causal the queries of a sequence are the last positions of its keys); out [T, Hq, 128] bf16; lse [Hq, T] fp32 or null.
extern "C" int vb_flash_fwd(const void* q, const void* k, const void* v, long long q_stride, long long k_stride,
                            long long v_stride, const int* cu_seqlens, const int* cu_k, int B, long long T, long long Tk,
                            int max_seqlen, int Hq, int Hk, float scale, int causal, void* out, long long out_stride,
                            float* lse, int* status, cudaStream_t stream) {
  if (B <= 0 || T <= 0 || max_seqlen <= 0) return 0;
  if (cu_k == nullptr) Tk = T;
  if (Hk <= 0 || Hq % Hk != 0 || (q_stride & 7) || (k_stride & 7) || (v_stride & 7) || (out_stride & 7)) return -3;
  CUtensorMap tmQ, tmK, tmV;
  int rc = vb_make_tmap_2d(&tmQ, q, 2, (uint64_t)Hq * FA_D, (uint64_t)T, (uint64_t)q_stride * 2, 64, FA_BM);
  if (rc) return rc;
  rc = vb_make_tmap_2d(&tmK, k, 2, (uint64_t)Hk * FA_D, (uint64_t)Tk, (uint64_t)k_stride * 2, 64, FA_BN);
  if (rc) return rc;
  rc = vb_make_tmap_2d(&tmV, v, 2, (uint64_t)Hk * FA_D, (uint64_t)Tk, (uint64_t)v_stride * 2, 64, FA_BN);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    VB_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM));
    attr_set = true;
  }
  FaParams p{};
  p.cu_seqlens = cu_seqlens;
  p.cu_k = cu_k;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.out_stride = out_stride;
  p.lse = lse;
  p.T = T;
  p.Hq = Hq; p.Hk = Hk;
  p.scale = scale;
  p.causal = causal;
  p.max_qblocks = (max_seqlen + FA_BM - 1) / FA_BM;
  p.status = status;
  dim3 grid(p.max_qblocks, Hq, B);
  flash_fwd_kernel<<<grid, FA_THREADS, FA_SMEM, stream>>>(tmQ, tmK, tmV, p);
  vb_count_launch();
  return (int)cudaGetLastError();
}
