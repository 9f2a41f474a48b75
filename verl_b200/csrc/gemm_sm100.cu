// Persistent warp-specialised bf16 GEMM for sm_100a built directly on tcgen05:
//   warp 0      : TMA producer (per-CTA 2-D tiled loads, 128-byte swizzle)
//   warp 1      : TMEM allocator + single-thread tcgen05.mma issuer
//   warps 2..5  : epilogue (tcgen05.ld from TMEM, one accumulator row per thread)
// The accumulator is double-buffered in TMEM (2 x BN fp32 columns) so the epilogue
// of tile i overlaps the main loop of tile i+1.
//
// One main loop serves several epilogues:
//   EPI_STORE   C = A.B^T (+bias) in bf16, or fp32 with optional C += (weight-gradient accumulation)
//   EPI_LSE     fused lm_head -> online-softmax statistics per row (no logits in memory);
//               role of verl/utils/kernel/kernels.py:183-343 (efficient_entropy_kernel_general_mainloop)
//   EPI_DLOGITS recompute the logits tile and emit d_logits in bf16;
//               role of verl/utils/kernel/kernels.py:1213-1509
//
// Operand layouts: an operand is "K-major" when the contraction index is contiguous
// in memory ([rows, K] row-major) and "MN-major" when the row index is contiguous
// ([K, rows] row-major). The forward pass of a Linear uses K-major/K-major, the data
// gradient K-major/MN-major, the weight gradient MN-major/MN-major; no transposes are
// materialised.
#include "common.cuh"
#include <cstdlib>
#include "host_utils.h"

namespace vb {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int GROUP_M = 8;

enum Epi : int { EPI_STORE = 0, EPI_LSE = 1, EPI_DLOGITS = 2, EPI_STORE_AG = 3 };
constexpr int AG_COPY_THREADS = 128;  // EPI_STORE_AG: four more warps pull the peers' shards of B
constexpr int AG_MAX_RANKS = 16;
constexpr int RS_STAGE_WARP_BYTES = 32 * 256;            // 32 rows x 128 bf16 columns per epilogue warp
constexpr int RS_STAGE_BYTES = 4 * RS_STAGE_WARP_BYTES + 16;

struct GemmParams {
  int M, N, K;
  // EPI_STORE
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;  // optional, length N
  int out_fp32;
  int accumulate;  // fp32 only: C += result
  // EPI_LSE / EPI_DLOGITS
  const long long* labels;  // [M]
  float inv_temperature;
  int num_splits;       // LSE: vocab splits per row block
  int nblk_per_split;   // LSE: N blocks per split
  float* partials;      // LSE: [M, num_splits, 4] = (max, sumexp, sum exp*logit, label logit)
  const float* row_lse;     // DLOGITS: [M] log-sum-exp of scaled logits
  const float* row_mean;    // DLOGITS: [M] E_p[logit]
  const float* g_logprob;   // DLOGITS: [M] dL/dlogprob
  const float* g_entropy;   // DLOGITS: [M] dL/dentropy (may be null)
  int n_offset;             // DLOGITS: vocab offset of this chunk (for label compare)
  // EPI_STORE split-K (k_splits > 1): every (tile, k slice) unit writes an fp32 partial tile to ws, the unit
  // that arrives last at the tile's ticket counter sums the slices in slice order and writes C
  int k_splits;
  int kb_per_split;
  float* ws;        // [k_splits, num_m * BM, num_n * BN] fp32
  int* counters;    // one per tile, zero before the launch and zero again after it
  // k_cluster != 0: the k_splits slices of a tile are the CTAs of one thread-block cluster (cluster size = k_splits,
  // one unit per CTA); the partial tiles stay in shared memory and are added up through distributed shared memory,
  // every CTA reducing and storing its share of the tile's rows. No workspace, no grid-wide barrier.
  int k_cluster;
  // EPI_STORE_AG: B = W [N, K] is assembled in ag_dst from the ranks' flat shards while the GEMM runs. Element e of
  // the sharded flat vector lives on rank e / ag_shard at offset e % ag_shard; W starts at element ag_w_off.
  // ag_ready[nb] counts the CTAs that have copied their slice of rows [nb*BN, (nb+1)*BN); a tile may load its B
  // operand once the count reaches the grid size.
  // Grouped GEMM (mixture-of-experts). grp_mode 1: the rows of A come in 128-row blocks, block b belongs to expert
  // grp_blk_expert[b] (< 0: unused block) and is multiplied by that expert's matrix, B = [E, N, K] (or [E, K, N]
  // for an MN-major B). grp_mode 2 (weight gradients): C = [E, M, N], unit (e, tile) contracts over the rows
  // [grp_off[e], grp_off[e+1]) of A and B (multiples of 64) and adds into C[e] (accumulate must be set).
  int grp_mode;
  int grp_E;
  const int* grp_blk_expert;
  const int* grp_off;
  // GEMM -> reduce-scatter (rs_rows > 0): output row r belongs to rank r / rs_rows and is stored at row r % rs_rows
  // of rs_dst[owner], this rank's slot in the owner's receive buffer (peer memory, plain stores over NVLink).
  void* rs_dst[AG_MAX_RANKS];
  int rs_rows;
  int rs_stage;  // bf16 tiles go through a per-warp shared-memory transpose so that a store instruction covers whole
                 // 256-byte row segments (uncoalesced 16-byte stores crawl over NVLink); needs RS_STAGE_BYTES more smem
  const void* ag_src[AG_MAX_RANKS];
  long long ag_shard;
  long long ag_w_off;
  __nv_bfloat16* ag_dst;
  unsigned* ag_ready;
  int* status;
};

template <int BN>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128) ? 6 : (BN == 64) ? 8 : 10;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], split-K reduce[2], tmem slot, abort flag, ticket
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 6) * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;  // slack for manual 1024-byte alignment
};

// Map a linear work index to (m block, first n block, number of n blocks).
struct Sched {
  int num_m, num_n, num_units, nblk_per_split, num_splits, k_splits, kb_per_split, num_kb;
  bool lse;
  __device__ Sched(const GemmParams& p, int BN, bool lse_) : lse(lse_) {
    num_m = (p.M + BM - 1) / BM;
    num_n = (p.N + BN - 1) / BN;
    num_kb = (p.K + BK - 1) / BK;
    k_splits = (!lse_ && p.k_splits > 1) ? p.k_splits : 1;
    kb_per_split = k_splits > 1 ? p.kb_per_split : num_kb;
    if (lse) {
      nblk_per_split = p.nblk_per_split;
      num_splits = p.num_splits;
      num_units = num_m * num_splits;
    } else {
      nblk_per_split = 1;
      num_splits = num_n;
      num_units = num_m * num_n * k_splits;
      if (p.grp_mode == 2) num_units *= p.grp_E;
    }
  }
  // k-block range [kb0, kb1) and k slice of unit u (the k slice is the fastest-varying part of u)
  __device__ void k_range(int u, int& ks, int& kb0, int& kb1) const {
    ks = u % k_splits;
    kb0 = ks * kb_per_split;
    kb1 = min(num_kb, kb0 + kb_per_split);
  }
  __device__ void get(int u, int& m_blk, int& n_first, int& n_count, int& split) const {
    u /= k_splits;
    const int per_group = GROUP_M * num_splits;
    const int g = u / per_group;
    const int first_m = g * GROUP_M;
    const int gsize = min(num_m - first_m, GROUP_M);
    const int r = u - g * per_group;
    m_blk = first_m + r % gsize;
    split = r / gsize;
    n_first = split * nblk_per_split;
    n_count = min(nblk_per_split, num_n - n_first);
  }
};

// Base pointer and row index for an output row: the local C, or the owner's receive slot for GEMM -> reduce-scatter.
__device__ __forceinline__ void* epi_row_base(const GemmParams& p, int& row) {
  if (p.rs_rows > 0) {
    const int owner = row / p.rs_rows;
    row -= owner * p.rs_rows;
    return p.rs_dst[owner];
  }
  return p.C;
}

// Final store of 32 consecutive columns of one output row (bias, fp32 accumulate or bf16 pack).
__device__ __forceinline__ void epi_store_chunk(const GemmParams& p, int row, int col0, uint32_t (&r)[32]) {
                void* const cbase = epi_row_base(p, row);
                if (p.bias != nullptr) {
  #pragma unroll
                  for (int i = 0; i < 32; ++i) {
                    if (col0 + i < p.N) r[i] = __float_as_uint(__uint_as_float(r[i]) + __bfloat162float(p.bias[col0 + i]));
                  }
                }
                if (p.out_fp32) {
                  float* dst = reinterpret_cast<float*>(cbase) + (long long)row * p.ldc + col0;
                  if (col0 + 32 <= p.N && (p.ldc & 3) == 0) {
  #pragma unroll
                    for (int i = 0; i < 8; ++i) {
                      float4 v = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                             __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
                      if (p.accumulate) {
                        float4 o = reinterpret_cast<float4*>(dst)[i];
                        v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                      }
                      reinterpret_cast<float4*>(dst)[i] = v;
                    }
                  } else {
  #pragma unroll
                    for (int i = 0; i < 32; ++i) {
                      if (col0 + i < p.N) {
                        float v = __uint_as_float(r[i]);
                        if (p.accumulate) v += dst[i];
                        dst[i] = v;
                      }
                    }
                  }
                } else {
                  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(cbase) + (long long)row * p.ldc + col0;
                  if (col0 + 32 <= p.N && (p.ldc & 7) == 0) {
  #pragma unroll
                    for (int i = 0; i < 4; ++i) {
                      uint4 v;
                      v.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
                      v.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
                      v.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
                      v.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
                      reinterpret_cast<uint4*>(dst)[i] = v;
                    }
                  } else {
  #pragma unroll
                    for (int i = 0; i < 32; ++i)
                      if (col0 + i < p.N) dst[i] = __float2bfloat16(__uint_as_float(r[i]));
                  }
                }
}

// Final store of 4 consecutive columns of one output row (split-K reduction).
__device__ __forceinline__ void epi_store4(const GemmParams& p, int row, int col, float4 v) {
  float x[4] = {v.x, v.y, v.z, v.w};
  const bool full = col + 4 <= p.N;
  void* const cbase = epi_row_base(p, row);
  if (p.bias != nullptr) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (col + i < p.N) x[i] += __bfloat162float(p.bias[col + i]);
  }
  if (p.out_fp32) {
    float* dst = reinterpret_cast<float*>(cbase) + (long long)row * p.ldc + col;
    if (full && (p.ldc & 3) == 0) {
      float4 o = make_float4(x[0], x[1], x[2], x[3]);
      if (p.accumulate) {
        const float4 old = *reinterpret_cast<const float4*>(dst);
        o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
      }
      *reinterpret_cast<float4*>(dst) = o;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (col + i < p.N) dst[i] = p.accumulate ? dst[i] + x[i] : x[i];
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(cbase) + (long long)row * p.ldc + col;
    if (full && (p.ldc & 3) == 0) {
      *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]));
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (col + i < p.N) dst[i] = __float2bfloat16(x[i]);
    }
  }
}


// Grouped-GEMM view of unit u: returns false when the unit has no work. On success `u` is the tile index inside the
// expert (mode 2), b_off the row offset of the expert's matrix in B, c_off the row offset of its output in C.
struct GroupView {
  int e, b_off, c_off, kb0, kb1;
};
template <bool B_MN>
__device__ __forceinline__ bool group_view(const GemmParams& p, const Sched& sched, int& u, GroupView& g) {
  g.e = 0; g.b_off = 0; g.c_off = 0; g.kb0 = -1; g.kb1 = -1;
  if (p.grp_mode == 2) {
    const int per_e = sched.num_m * sched.num_n;
    g.e = u / per_e;
    u -= g.e * per_e;
    g.kb0 = p.grp_off[g.e] / BK;
    g.kb1 = p.grp_off[g.e + 1] / BK;
    g.c_off = g.e * p.M;
    return g.kb1 > g.kb0;
  }
  return true;
}
template <bool B_MN>
__device__ __forceinline__ bool group_rows(const GemmParams& p, int m_blk, GroupView& g) {
  if (p.grp_mode == 1) {
    g.e = p.grp_blk_expert[m_blk];
    if (g.e < 0) return false;
    g.b_off = g.e * (B_MN ? p.K : p.N);
  }
  return true;
}

template <int BN, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(EPI == EPI_STORE_AG ? NUM_THREADS + AG_COPY_THREADS : NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  using L = SmemLayout<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smemA = smem;
  uint8_t* smemB = smem + L::STAGES * L::A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty = full + L::STAGES;
  uint64_t* tfull = empty + L::STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* rbar = tempty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(rbar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* ticket_s = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const Sched sched(p, BN, EPI == EPI_LSE);
  vb_jitter(100u);

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
      mbar_init(&rbar[a], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();  // TMEM is held: a dependent kernel may take what is left
  pdl_wait();     // nothing above reads or writes global memory

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int uu = blockIdx.x; ok && uu < sched.num_units; uu += gridDim.x) {
        int u = uu;
        GroupView gv;
        if (!group_view<B_MN>(p, sched, u, gv)) continue;
        int m_blk, n_first, n_count, split;
        sched.get(u, m_blk, n_first, n_count, split);
        if (!group_rows<B_MN>(p, m_blk, gv)) continue;
        int ks, kb0, kb1;
        sched.k_range(u, ks, kb0, kb1);
        if (gv.kb0 >= 0) { kb0 = gv.kb0; kb1 = gv.kb1; }
        for (int nb = n_first; ok && nb < n_first + n_count; ++nb) {
          if (EPI == EPI_STORE_AG) {
            // rows [nb*BN, (nb+1)*BN) of B must have arrived from all ranks (every CTA copies a slice of them)
            const uint64_t t0 = globaltimer_ns();
            uint32_t spins = 0;
            while (true) {
              unsigned v;
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.ag_ready + nb) : "memory");
              if (v >= gridDim.x) break;
              if ((++spins & 0xff) == 0 && (*abort_flag || globaltimer_ns() - t0 > VB_WAIT_LIMIT_NS)) {
                report_error(p.status, ERR_WAIT_FLAG, nb);
                *abort_flag = 1;
                ok = false;
                break;
              }
            }
            if (!ok) break;
            asm volatile("fence.proxy.async.global;" ::: "memory");  // generic-proxy copies -> TMA reads
          }
          for (int kb = kb0; kb < kb1; ++kb) {
            if (*abort_flag || !mbar_wait(&empty[s], phase ^ 1)) {
              report_error(p.status, ERR_WAIT_EMPTY, kb);
              *abort_flag = 1;
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&full[s], L::STAGE_BYTES);
            uint8_t* a_dst = smemA + s * L::A_BYTES;
            uint8_t* b_dst = smemB + s * L::B_BYTES;
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                tma_load_2d(a_dst + j * (BK * 128), &tmA, &full[s], m_blk * BM + j * 64, kb * BK);
            } else {
              tma_load_2d(a_dst, &tmA, &full[s], kb * BK, m_blk * BM);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(b_dst + j * (BK * 128), &tmB, &full[s], nb * BN + j * 64, gv.b_off + kb * BK);
            } else {
              tma_load_2d(b_dst, &tmB, &full[s], kb * BK, gv.b_off + nb * BN);
            }
            if (++s == L::STAGES) {
              s = 0;
              phase ^= 1;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0, BM, BN);
      int s = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int uu = blockIdx.x; ok && uu < sched.num_units; uu += gridDim.x) {
        int u = uu;
        GroupView gv;
        if (!group_view<B_MN>(p, sched, u, gv)) continue;
        int m_blk, n_first, n_count, split;
        sched.get(u, m_blk, n_first, n_count, split);
        if (!group_rows<B_MN>(p, m_blk, gv)) continue;
        int ks, kb0, kb1;
        sched.k_range(u, ks, kb0, kb1);
        if (gv.kb0 >= 0) { kb0 = gv.kb0; kb1 = gv.kb1; }
        for (int nb = n_first; ok && nb < n_first + n_count; ++nb) {
          if (*abort_flag || !mbar_wait(&tempty[acc], acc_phase ^ 1)) {
            report_error(p.status, ERR_WAIT_TMEM_EMPTY, nb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BN;
          for (int kb = kb0; kb < kb1; ++kb) {
            if (*abort_flag || !mbar_wait(&full[s], phase)) {
              report_error(p.status, ERR_WAIT_FULL, kb);
              *abort_flag = 1;
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a_addr = smem_u32(smemA + s * L::A_BYTES);
            const uint32_t b_addr = smem_u32(smemB + s * L::B_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t a_desc = A_MN ? umma_smem_desc(a_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                           : umma_smem_desc(a_addr + k * (UMMA_K * 2), 16, 1024);
              const uint64_t b_desc = B_MN ? umma_smem_desc(b_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                           : umma_smem_desc(b_addr + k * (UMMA_K * 2), 16, 1024);
              tc_mma_f16(d_tmem, a_desc, b_desc, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
            }
            tc_commit(&empty[s]);  // frees the stage once these MMAs have read it
            if (++s == L::STAGES) {
              s = 0;
              phase ^= 1;
            }
          }
          if (!ok) break;
          tc_commit(&tfull[acc]);
          if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1;
          }
        }
      }
    }
  } else if (EPI == EPI_STORE_AG && warp >= 6) {
    // ------------------------------ all-gather of B (copy warps) ----------------------------------
    // Chunk after chunk, in the order in which the tiles need them, every CTA copies 1/gridDim of the chunk from
    // the ranks that own it (plain 16-byte loads over NVLink for remote ranks) into the local full matrix.
    const int ct = threadIdx.x - NUM_THREADS;
    const int num_n = (p.N + BN - 1) / BN;
    uint4* dst = reinterpret_cast<uint4*>(p.ag_dst);
    const long long shard16 = p.ag_shard >> 3, off16 = p.ag_w_off >> 3, row16 = (long long)p.K >> 3;
    for (int j = 0; j < num_n; ++j) {
      const long long c_lo = (long long)j * BN * row16;
      const long long c_hi = min((long long)(j + 1) * BN, (long long)p.N) * row16;
      const long long per = (c_hi - c_lo + gridDim.x - 1) / gridDim.x;
      const long long lo = c_lo + (long long)blockIdx.x * per;
      const long long hi = min(lo + per, c_hi);
      constexpr int U = 8;
      for (long long i0 = lo + ct; i0 < hi; i0 += (long long)AG_COPY_THREADS * U) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + (long long)u * AG_COPY_THREADS;
          if (i < hi) {
            const long long e = off16 + i;
            const int r = (int)(e / shard16);
            v[u] = reinterpret_cast<const uint4*>(p.ag_src[r])[e - (long long)r * shard16];
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + (long long)u * AG_COPY_THREADS;
          if (i < hi) dst[i] = v[u];
        }
      }
      __threadfence();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (ct == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.ag_ready + j) : "memory");
    }
  } else if (warp < 6) {
    // ------------------------------ epilogue ----------------------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int uu = blockIdx.x; ok && uu < sched.num_units; uu += gridDim.x) {
      int u = uu;
      GroupView gv;
      if (!group_view<B_MN>(p, sched, u, gv)) continue;
      int m_blk, n_first, n_count, split;
      sched.get(u, m_blk, n_first, n_count, split);
      if (!group_rows<B_MN>(p, m_blk, gv)) continue;
      int ks, kb0, kb1;
      sched.k_range(u, ks, kb0, kb1);
      const bool row_ok = m_blk * BM + row_in_tile < p.M;
      const int row = gv.c_off + m_blk * BM + row_in_tile;  // grouped weight gradients: row inside C = [E * M, N]

      // per-row state for the fused epilogues
      float run_max = -INFINITY, run_sum = 0.f, run_dot = 0.f, label_logit = 0.f;
      long long label = -1;
      float r_lse = 0.f, r_mean = 0.f, r_glp = 0.f, r_gent = 0.f;
      if (EPI == EPI_LSE || EPI == EPI_DLOGITS) {
        if (row_ok) label = p.labels[row];
      }
      if (EPI == EPI_DLOGITS) {
        if (row_ok) {
          r_lse = p.row_lse[row];
          r_mean = p.row_mean[row];
          r_glp = p.g_logprob[row];
          r_gent = p.g_entropy ? p.g_entropy[row] : 0.f;
        }
      }

      for (int nb = n_first; ok && nb < n_first + n_count; ++nb) {
        if (*abort_flag || !mbar_wait(&tfull[acc], acc_phase)) {
          report_error(p.status, ERR_WAIT_TMEM_FULL, nb);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait();
          const int col0 = nb * BN + c * 32;
          if (EPI == EPI_STORE || EPI == EPI_STORE_AG) {
            if (sched.k_splits > 1 && p.k_cluster) {
              // fp32 partial tile into the (now idle) pipeline stages: [BM rows][BN / 4 float4], the float4 index
              // XOR-swizzled by the row so that the 32 rows of a warp do not hit the same banks
              float4* stg = reinterpret_cast<float4*>(smem);
              constexpr int SWZ = (BN / 4 >= 32) ? 31 : (BN / 4 - 1);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int j = c * 8 + i;
                stg[row_in_tile * (BN / 4) + (j ^ (row_in_tile & SWZ))] =
                    make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]),
                                __uint_as_float(r[4 * i + 3]));
              }
            } else if (sched.k_splits > 1) {
              // fp32 partial: slice ks of the padded [num_m * BM, num_n * BN] output
              float4* dst = reinterpret_cast<float4*>(
                  p.ws + ((long long)ks * sched.num_m * BM + row) * ((long long)sched.num_n * BN) + col0);
#pragma unroll
              for (int i = 0; i < 8; ++i)
                __stcg(dst + i, make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                            __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3])));
            } else if (p.rs_stage) {
              // GEMM -> reduce-scatter over NVLink: transpose 128-column groups through shared memory, then every
              // store instruction of the warp writes two whole 256-byte row segments of the owner's slot
              uint8_t* stg = smem + ((L::TOTAL + 15) & ~15) + quad * RS_STAGE_WARP_BYTES;
              const int cl = c & 3;
              if (p.bias != nullptr) {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (col0 + i < p.N) r[i] = __float_as_uint(__uint_as_float(r[i]) + __bfloat162float(p.bias[col0 + i]));
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
                v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
                const int piece = cl * 4 + j;
                *reinterpret_cast<uint4*>(stg + lane * 256 + ((piece ^ (lane & 15)) << 4)) = v;
              }
              if (cl == 3 || c == BN / 32 - 1) {
                __syncwarp();
                const int col_base = nb * BN + (c - cl) * 32;
                const int pieces = (cl + 1) * 4;
#pragma unroll 4
                for (int i = 0; i < 16; ++i) {
                  const int idx = i * 32 + lane;
                  const int rr = idx >> 4, piece = idx & 15;
                  const int grow = m_blk * BM + quad * 32 + rr, gcol = col_base + piece * 8;
                  if (piece < pieces && grow < p.M && gcol < p.N) {
                    const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 256 + ((piece ^ (rr & 15)) << 4));
                    const int owner = grow / p.rs_rows;
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.rs_dst[owner]) +
                                         (long long)(grow - owner * p.rs_rows) * p.ldc + gcol;
                    *reinterpret_cast<uint4*>(dst) = v;
                  }
                }
                __syncwarp();
              }
            } else if (row_ok && col0 < p.N) {
              epi_store_chunk(p, row, col0, r);
            }
          } else if (EPI == EPI_LSE) {
            if (col0 < p.N) {
              float cmax = -INFINITY;
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                float x = __uint_as_float(r[i]) * p.inv_temperature;
                x = (col0 + i < p.N) ? x : -INFINITY;
                if ((long long)(col0 + i) == label) label_logit = x;
                r[i] = __float_as_uint(x);
                cmax = fmaxf(cmax, x);
              }
              const float new_max = fmaxf(run_max, cmax);
              const float scale = __expf(run_max - new_max);  // exp(-inf) = 0 on the first chunk
              float csum = 0.f, cdot = 0.f;
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float x = __uint_as_float(r[i]);
                const float e = __expf(x - new_max);  // exp(-inf) = 0 for masked columns
                csum += e;
                cdot += (col0 + i < p.N) ? e * x : 0.f;
              }
              run_sum = run_sum * scale + csum;
              run_dot = run_dot * scale + cdot;
              run_max = new_max;
            }
          } else {  // EPI_DLOGITS
            if (row_ok && col0 < p.N) {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
              const long long rel = label - (long long)p.n_offset - col0;
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float x = __uint_as_float(r[i]) * p.inv_temperature;
                const float pr = __expf(x - r_lse);
                float g = r_glp * (((long long)i == rel ? 1.f : 0.f) - pr) - r_gent * pr * (x - r_mean);
                r[i] = __float_as_uint(g * p.inv_temperature);
              }
              if (col0 + 32 <= p.N && (p.ldc & 7) == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  uint4 v;
                  v.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
                  v.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
                  v.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
                  v.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
                  reinterpret_cast<uint4*>(dst)[i] = v;
                }
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (col0 + i < p.N) dst[i] = __float2bfloat16(__uint_as_float(r[i]));
              }
            }
          }
        }
        // release this accumulator buffer to the MMA warp
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
      if (EPI == EPI_STORE || EPI == EPI_STORE_AG) {
        if (sched.k_splits > 1 && !p.k_cluster) {
          // All units have written their fp32 slice. After a grid-wide barrier (the launch is cooperative and every
          // CTA owns exactly one unit) EVERY CTA reduces an equal share of the output: its share of each slice comes
          // back through one bulk async copy into the idle pipeline stages, the slices are summed in slice order
          // (deterministic) and stored. counters[0] = arrivals, counters[1] = departures; the last CTA to leave
          // zeroes both for the next launch.
          const int et = threadIdx.x - 64;
          const int S = sched.k_splits;
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (et == 0) {
            atomicAdd(reinterpret_cast<unsigned*>(p.counters), 1u);
            const uint64_t t0 = globaltimer_ns();
            uint32_t spins = 0;
            int good = ok ? 1 : 0;
            while (true) {
              unsigned v;
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.counters) : "memory");
              if (v >= gridDim.x) break;
              if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > VB_WAIT_LIMIT_NS) {
                report_error(p.status, ERR_WAIT_FLAG, 3000);
                good = 0;
                break;
              }
            }
            *ticket_s = good;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const bool go = *ticket_s != 0;
          if (go) {
            asm volatile("fence.proxy.async.global;" ::: "memory");
            const long long ldw4 = (long long)sched.num_n * BN / 4;            // float4 per padded row
            const long long slice4 = (long long)sched.num_m * BM * ldw4;       // float4 per slice
            const long long per = (slice4 + gridDim.x - 1) / gridDim.x;
            const long long lo = (long long)blockIdx.x * per, hi = min(lo + per, slice4);
            const int cap = (SmemLayout<BN>::BAR_OFFSET / 16) / S;              // float4 of one slice per round
            const float4* ws4 = reinterpret_cast<const float4*>(p.ws);
            float4* buf = reinterpret_cast<float4*>(smem);
            uint32_t rphase = 0;
            for (long long r0 = lo; r0 < hi; r0 += cap) {
              const int n = (int)min((long long)cap, hi - r0);
              if (et == 0) {
                mbar_arrive_expect_tx(&rbar[0], (uint32_t)(S * n * 16));
                for (int sp = 0; sp < S; ++sp) bulk_load(buf + (long long)sp * n, ws4 + sp * slice4 + r0, n * 16, &rbar[0]);
              }
              if (!mbar_wait(&rbar[0], rphase)) {
                report_error(p.status, ERR_WAIT_FULL, 2000);
                break;
              }
              rphase ^= 1;
              for (int i = et; i < n; i += 128) {
                float4 acc = buf[i];
                for (int sp = 1; sp < S; ++sp) {
                  const float4 v = buf[sp * n + i];
                  acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                }
                const long long f = r0 + i;
                const int orow = (int)(f / ldw4), ocol = (int)(f % ldw4) * 4;
                if (orow < p.M && ocol < p.N) epi_store4(p, orow, ocol, acc);
              }
              asm volatile("bar.sync 1, 128;" ::: "memory");  // the staging area is free for the next round
            }
          }
          if (et == 0) {
            const unsigned left = atomicAdd(reinterpret_cast<unsigned*>(p.counters) + 1, 1u);
            if (left == gridDim.x - 1) {
              p.counters[0] = 0;
              p.counters[1] = 0;
            }
          }
        }
      }
      if (EPI == EPI_LSE) {
        if (ok && row_ok) {
          float4 out = make_float4(run_max, run_sum, run_dot, label_logit);
          reinterpret_cast<float4*>(p.partials)[(long long)row * p.num_splits + split] = out;
        }
      }
    }
  }

  if (EPI == EPI_STORE && p.k_cluster && sched.k_splits > 1) {
    // Split-K inside a cluster: every CTA has left its fp32 partial tile in its own shared memory. After a cluster
    // barrier CTA r adds up rows [r * rows_per, (r + 1) * rows_per) of all CTAs' tiles (slice order: deterministic)
    // through distributed shared memory and stores them; a second barrier keeps every CTA's shared memory alive
    // until its peers have read it. All threads of the CTA take part in both barriers.
    cluster_sync_all();
    if (warp >= 2 && warp < 6) {
      const int et = threadIdx.x - 64;
      const int S = sched.k_splits;
      const int cr = (int)cluster_ctarank();
      int m_blk, n_first, n_count, split;
      sched.get((int)blockIdx.x, m_blk, n_first, n_count, split);
      const int rows_per = (BM + S - 1) / S;
      const int r0 = cr * rows_per, r1 = min(BM, r0 + rows_per);
      constexpr int Q4 = BN / 4;
      constexpr int SWZ = (Q4 >= 32) ? 31 : (Q4 - 1);
      const float4* stg = reinterpret_cast<const float4*>(smem);
      for (int idx = et; idx < (r1 - r0) * Q4; idx += 128) {
        const int rr = r0 + idx / Q4, j = idx % Q4;
        const uint32_t local = smem_u32(stg + rr * Q4 + (j ^ (rr & SWZ)));
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sp = 0; sp < S; ++sp) {
          const uint32_t remote = map_to_cta(local, (uint32_t)sp);
          float4 v;
          asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                       : "r"(remote)
                       : "memory");
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        const int grow = m_blk * BM + rr, gcol = n_first * BN + j * 4;
        if (grow < p.M && gcol < p.N) epi_store4(p, grow, gcol, acc);
      }
    }
    cluster_sync_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// Merge the per-split statistics of the fused lm_head kernel.
// Role of verl/utils/kernel/kernels.py:346-435 (efficient_entropy_triton_kernel_epilogue).
__global__ void lse_merge_kernel(const float4* __restrict__ partials, int M, int num_splits,
                                 float* __restrict__ logprob, float* __restrict__ entropy, float* __restrict__ lse_out,
                                 float* __restrict__ mean_out) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  float m = -INFINITY, s = 0.f, d = 0.f, ll = 0.f;
  for (int i = 0; i < num_splits; ++i) {
    const float4 v = partials[(long long)row * num_splits + i];
    const float nm = fmaxf(m, v.x);
    const float a = __expf(m - nm), b = __expf(v.x - nm);
    s = s * a + v.y * b;
    d = d * a + v.z * b;
    m = nm;
    ll += v.w;
  }
  const float lse = m + logf(s);
  const float mean = d / s;
  if (logprob) logprob[row] = ll - lse;
  if (entropy) entropy[row] = lse - mean;
  if (lse_out) lse_out[row] = lse;
  if (mean_out) mean_out[row] = mean;
}

// ---------------------------------------------------------------------------------------------------
// CTA-pair GEMM (cta_group::2): a cluster of two CTAs owns a 256 x 256 output tile. Each CTA stages its own
// 128 rows of A and its own 128 of the 256 columns' rows of B (32 KB per stage instead of 48 KB, six stages),
// CTA 0 issues one 256 x 256 x 16 MMA for both, and each CTA drains its 128 accumulator rows from its own TMEM.
// Barrier protocol (all barriers at the same shared-memory offset in both CTAs):
//   full[s]    lives in CTA 0, count 2: each CTA's producer arrives with its own byte count; both CTAs' TMA
//              loads report their bytes there
//   empty[s]   CTA 0: arrived by tcgen05.commit; CTA 1: arrived by CTA 0's producer after it saw that commit
//   tfull[a]   CTA 0: tcgen05.commit after the last k block; CTA 1: relayed by CTA 0's first epilogue warp
//   tempty[a]  lives in CTA 0, count 8: the four epilogue warps of both CTAs
// No load in this kernel is shared between CTAs: every CTA fetches exactly the bytes it owns.
constexpr int P_BN = 256;
constexpr int P_STAGES = 6;
constexpr int P_A_BYTES = BM * BK * 2;          // 16 KB
constexpr int P_B_BYTES = (P_BN / 2) * BK * 2;  // 16 KB
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int P_BAR_OFFSET = P_STAGES * P_STAGE_BYTES;
constexpr int P_DYN_BYTES = P_BAR_OFFSET + (2 * P_STAGES + 4) * 8 + 16 + 1024;

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smemA = smem;
  uint8_t* smemB = smem + P_STAGES * P_A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + P_BAR_OFFSET);
  uint64_t* empty = full + P_STAGES;
  uint64_t* tfull = empty + P_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 issues the MMAs
  const int num_m2 = (p.M + 2 * BM - 1) / (2 * BM);
  const int num_n = (p.N + P_BN - 1) / P_BN;
  const int num_units = num_m2 * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  const int first_unit = (int)cluster_id_x();
  const int unit_stride = (int)cluster_nctaid_x();
  // unit -> (256-row block, 256-column block); row blocks grouped so that neighbouring clusters share B in L2
  auto unit_coords = [&](int u, int& m2, int& nb) {
    const int per_group = GROUP_M * num_n;
    const int g = u / per_group;
    const int first_m = g * GROUP_M;
    const int gsize = min(num_m2 - first_m, GROUP_M);
    const int r = u - g * per_group;
    m2 = first_m + r % gsize;
    nb = r / gsize;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&full[s], 2);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 2 * P_BN);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised and both allocations are done
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();  // TMEM is held: a dependent kernel may take what is left
  pdl_wait();     // nothing above reads or writes global memory

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int s = 0;
      uint32_t phase = 0;
      int round = 0;
      bool ok = true;
      for (int u = first_unit; ok && u < num_units; u += unit_stride) {
        int m2, nb;
        unit_coords(u, m2, nb);
        const int m0 = (2 * m2 + (int)rank) * BM;
        const int n0 = nb * P_BN + (int)rank * (P_BN / 2);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (*abort_flag || !mbar_wait(&empty[s], phase ^ 1)) {
            report_error(p.status, ERR_WAIT_EMPTY, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          // CTA 0 saw the commit that frees stage s in both CTAs: pass it on (not in the first round, where
          // nothing had to be freed)
          if (rank == 0 && round > 0) mbar_arrive_cluster(map_to_cta(smem_u32(&empty[s]), 1));
          const uint32_t full0 = map_to_cta(smem_u32(&full[s]), 0);
          mbar_arrive_expect_tx_cluster(full0, P_STAGE_BYTES);
          uint8_t* a_dst = smemA + s * P_A_BYTES;
          uint8_t* b_dst = smemB + s * P_B_BYTES;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(a_dst + j * (BK * 128), &tmA, full0, m0 + j * 64, kb * BK);
          } else {
            tma_load_2d_pair(a_dst, &tmA, full0, kb * BK, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < P_BN / 2 / 64; ++j)
              tma_load_2d_pair(b_dst + j * (BK * 128), &tmB, full0, n0 + j * 64, kb * BK);
          } else {
            tma_load_2d_pair(b_dst, &tmB, full0, kb * BK, n0);
          }
          if (++s == P_STAGES) {
            s = 0;
            phase ^= 1;
            ++round;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (CTA 0 only) --------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc(1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0, 2 * BM, P_BN);
      int s = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int u = first_unit; ok && u < num_units; u += unit_stride) {
        if (*abort_flag || !mbar_wait(&tempty[acc], acc_phase ^ 1)) {
          report_error(p.status, ERR_WAIT_TMEM_EMPTY, u);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * P_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (*abort_flag || !mbar_wait(&full[s], phase)) {
            report_error(p.status, ERR_WAIT_FULL, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smemA + s * P_A_BYTES);
          const uint32_t b_addr = smem_u32(smemB + s * P_B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t a_desc = A_MN ? umma_smem_desc(a_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                         : umma_smem_desc(a_addr + k * (UMMA_K * 2), 16, 1024);
            const uint64_t b_desc = B_MN ? umma_smem_desc(b_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                         : umma_smem_desc(b_addr + k * (UMMA_K * 2), 16, 1024);
            tc_mma_f16_pair(d_tmem, a_desc, b_desc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit_pair(&empty[s]);
          if (++s == P_STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        tc_commit_pair(&tfull[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ----------------------------------
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int u = first_unit; ok && u < num_units; u += unit_stride) {
      int m2, nb;
      unit_coords(u, m2, nb);
      const int row = (2 * m2 + (int)rank) * BM + row_in_tile;
      const bool row_ok = row < p.M;
      if (*abort_flag || !mbar_wait(&tfull[acc], acc_phase)) {
        report_error(p.status, ERR_WAIT_TMEM_FULL, u);
        *abort_flag = 1;
        ok = false;
        break;
      }
      if (rank == 0 && warp == 2 && lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tfull[acc]), 1));
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * P_BN;
#pragma unroll 1
      for (int c = 0; c < P_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = nb * P_BN + c * 32;
        if (row_ok && col0 < p.N) epi_store_chunk(p, row, col0, r);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty[acc]), 0));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the other CTA may still read this CTA's shared memory or signal its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 2 * P_BN);
  }
}

template <bool A_MN, bool B_MN>
static int launch_gemm_pair(const void* A, const void* B, long long lda, long long ldb, const GemmParams& p,
                            cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  int rc;
  if (A_MN) rc = vb_make_tmap_2d(&tmA, A, 2, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)lda * 2, 64, BK);
  else rc = vb_make_tmap_2d(&tmA, A, 2, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)lda * 2, BK, BM);
  if (rc) return rc;
  if (B_MN) rc = vb_make_tmap_2d(&tmB, B, 2, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)ldb * 2, 64, BK);
  else rc = vb_make_tmap_2d(&tmB, B, 2, (uint64_t)p.K, (uint64_t)p.N, (uint64_t)ldb * 2, BK, P_BN / 2);
  if (rc) return rc;
  auto kern = gemm_pair_kernel<A_MN, B_MN>;
  static int max_clusters = 0;  // clusters of two that the device can hold at once (per instantiation)
  if (max_clusters == 0) {
    VB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_DYN_BYTES));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (vb_num_sms() / 2));
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = P_DYN_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = -1;
    }
    max_clusters = n;
  }
  if (max_clusters < 0) return -7;
  const int units = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + P_BN - 1) / P_BN);
  if (units <= 0) return 0;
  const int clusters = units < max_clusters ? units : max_clusters;
  cudaError_t e = vb_launch_pdl(kern, dim3(2 * clusters), dim3(NUM_THREADS), P_DYN_BYTES, stream, 1, tmA, tmB, p);
  vb_count_launch();
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

template <int BN, bool A_MN, bool B_MN, int EPI>
static int launch_gemm(const void* A, const void* B, long long lda, long long ldb, const GemmParams& p,
                       cudaStream_t stream) {
  using L = SmemLayout<BN>;
  CUtensorMap tmA, tmB;
  int rc;
  if (A_MN) rc = vb_make_tmap_2d(&tmA, A, 2, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)lda * 2, 64, BK);
  else rc = vb_make_tmap_2d(&tmA, A, 2, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)lda * 2, BK, BM);
  if (rc) return rc;
  if (B_MN) rc = vb_make_tmap_2d(&tmB, B, 2, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)ldb * 2, 64, BK);
  else rc = vb_make_tmap_2d(&tmB, B, 2, (uint64_t)p.K, (uint64_t)p.N, (uint64_t)ldb * 2, BK, BN);
  if (rc) return rc;
  auto kern = gemm_kernel<BN, A_MN, B_MN, EPI>;
  constexpr bool can_stage = EPI == EPI_STORE && BN >= 64;  // room for the reduce-scatter staging area
  if (p.rs_stage && !can_stage) return -3;
  const int dyn_bytes = L::DYN_BYTES + (p.rs_stage ? RS_STAGE_BYTES : 0);
  static bool attr_set = false;
  if (!attr_set) {
    VB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       L::DYN_BYTES + (can_stage ? RS_STAGE_BYTES : 0)));
    attr_set = true;
  }
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int units = (EPI == EPI_LSE) ? num_m * p.num_splits : num_m * num_n * (p.k_splits > 1 ? p.k_splits : 1);
  if (units <= 0) return 0;
  const int grid = units < vb_num_sms() ? units : vb_num_sms();
  // kernels that wait on other ranks (all-gather prologue, reduce-scatter epilogue) start the ordinary way
  const bool pdl = EPI != EPI_STORE_AG && p.rs_rows == 0;
  if (EPI == EPI_STORE && p.k_splits > 1 && p.k_cluster) {
    // one cluster per output tile, one CTA per k slice; clusters are scheduled as SMs free up (no grid-wide barrier)
    cudaError_t e = vb_launch_ex(kern, dim3(units), dim3(NUM_THREADS), dyn_bytes, stream, (unsigned)p.k_splits, pdl,
                                 tmA, tmB, p);
    vb_count_launch();
    return (int)e;
  }
  if (EPI == EPI_STORE && p.k_splits > 1) {
    // the split-K reduction has a grid-wide barrier: every CTA owns one unit and all of them must be resident
    if (units > vb_num_sms()) return -3;
    void* args[] = {(void*)&tmA, (void*)&tmB, (void*)&p};
    cudaError_t e = cudaLaunchCooperativeKernel((const void*)kern, dim3(units), dim3(NUM_THREADS), args, dyn_bytes, stream);
    if (e != cudaSuccess) {
      // e.g. a capture mode that refuses cooperative nodes: a plain launch of at most one CTA per SM is resident as
      // a whole on an otherwise idle device, and the barrier's wait is bounded in any case
      (void)cudaGetLastError();
      kern<<<units, NUM_THREADS, dyn_bytes, stream>>>(tmA, tmB, p);
      e = cudaGetLastError();
    }
    vb_count_launch();
    return (int)e;
  }
  cudaError_t e = vb_launch_ex(kern, dim3(grid), dim3(NUM_THREADS), dyn_bytes, stream, 1, pdl, tmA, tmB, p);
  vb_count_launch();
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}


// Number of clusters of `cluster` CTAs of the plain-store GEMM kernel with BN-wide tiles that the device can hold at
// once (one CTA per SM because of its shared memory; a cluster must fit inside one GPC). Cached; 0 if the query fails.
static int max_active_clusters(int bn, int cluster) {
  static int cache[2][9];
  static bool init = false;
  if (!init) {
    for (auto& row : cache)
      for (int& v : row) v = -1;
    init = true;
  }
  if (cluster < 1 || cluster > 8 || (bn != 128 && bn != 64)) return 0;
  int& slot = cache[bn == 128 ? 0 : 1][cluster];
  if (slot >= 0) return slot;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(cluster * 64);
  cfg.blockDim = dim3(NUM_THREADS);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  cudaError_t e;
  if (bn == 128) {
    auto kern = gemm_kernel<128, false, false, EPI_STORE>;
    cfg.dynamicSmemBytes = SmemLayout<128>::DYN_BYTES;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout<128>::DYN_BYTES + RS_STAGE_BYTES);
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
  } else {
    auto kern = gemm_kernel<64, false, false, EPI_STORE>;
    cfg.dynamicSmemBytes = SmemLayout<64>::DYN_BYTES;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout<64>::DYN_BYTES + RS_STAGE_BYTES);
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
  }
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    n = 0;
  }
  slot = n;
  return n;
}

}  // namespace vb

using namespace vb;

// C[M,N] = A . B^T, bf16 inputs, fp32 accumulation.
//   a_mn = 0: A is [M,K] row-major (lda elements per row); a_mn = 1: A is stored [K,M] row-major.
//   b_mn = 0: B is [N,K] row-major;                         b_mn = 1: B is stored [K,N] row-major.
//   out_fp32 = 0: C bf16; 1: C fp32, and accumulate != 0 adds into C.
// Requirements: lda, ldb multiples of 8; pointers 16-byte aligned.
//
// ws / counters (optional): fp32 workspace of ws_bytes and num_counters zeroed ints that enable split-K for
// problems with too few output tiles to occupy the GPU (decode-time projections: M <= 128, large K). Calls
// that share a workspace must be ordered on one stream. The counters are left at zero.
static int gemm_bf16_run(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                         long long lda, long long ldb, long long ldc, int a_mn, int b_mn, int out_fp32,
                         int accumulate, float* ws, long long ws_bytes, int* counters, int num_counters,
                         int* status, cudaStream_t stream, void* const* rs_dst, int rs_world, int rs_rows) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7)) return -3;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.out_fp32 = out_fp32; p.accumulate = accumulate; p.status = status;
  p.k_splits = 1;
  if (rs_dst != nullptr) {
    if (rs_world < 1 || rs_world > AG_MAX_RANKS || rs_rows <= 0 || (long long)rs_rows * rs_world < M || accumulate)
      return -3;
    for (int r = 0; r < rs_world; ++r) p.rs_dst[r] = rs_dst[r];
    p.rs_rows = rs_rows;
    // bf16 tiles of non-skinny problems take the coalescing path (single-CTA kernel, tiles 128 or 256 wide)
    p.rs_stage = (!out_fp32 && M > 256 && N >= 128 && (N & 7) == 0 && (ldc & 7) == 0) ? 1 : 0;
  }
  static const int splitk_mode = []() {
    const char* e = getenv("VERL_B200_SPLITK");  // 0 = never split K, N > 1 = force that many slices (experiments)
    return e ? atoi(e) : -1;
  }();
  static const bool cluster_sk = []() {
    const char* e = getenv("VERL_B200_SPLITK_CLUSTER");  // 0 = workspace + grid-barrier reduction (the older path)
    return !(e && e[0] == '0');
  }();
  if (cluster_sk && splitk_mode != 0 && !accumulate && N > 128) {
    // Skinny problems (decode projections): split K over the CTAs of a cluster and reduce through distributed shared
    // memory. Among tile widths {128, 64} and cluster sizes 2..8 take the pair that puts the most CTAs to work in ONE
    // wave: a cluster needs all its SMs free inside one GPC at once, so the number of co-resident clusters (asked
    // from the occupancy calculator, cached) bounds the tile count; a second wave would cost more than it gains.
    const int nm = (M + BM - 1) / BM, nkb = (K + BK - 1) / BK;
    int best_bn = 0, best_s = 0, best_ctas = 0;
    for (int bi = 0; bi < 2; ++bi) {
      const int bn = bi == 0 ? 128 : 64;
      const int tiles = nm * ((N + bn - 1) / bn);
      for (int sp = 2; sp <= 8; ++sp) {
        if (sp > nkb / 4) break;
        if (splitk_mode > 1 && sp != (splitk_mode > 8 ? 8 : splitk_mode)) continue;
        const int per = (nkb + sp - 1) / sp;
        if ((nkb + per - 1) / per != sp) continue;  // this slice count leaves an empty slice
        const int ctas = tiles * sp;
        if (ctas > vb_num_sms() || ctas <= best_ctas) continue;
        if (tiles > max_active_clusters(bn, sp)) continue;
        best_bn = bn; best_s = sp; best_ctas = ctas;
      }
    }
    // worth it only when it beats what plain tiling puts to work
    const int plain_ctas = nm * ((N + 31) / 32) < vb_num_sms() ? nm * ((N + 31) / 32) : vb_num_sms();
    if (best_s >= 2 && (best_ctas * 5 >= vb_num_sms() * 3 || best_ctas > plain_ctas)) {
      p.k_splits = best_s;
      p.kb_per_split = (nkb + best_s - 1) / best_s;
      p.k_cluster = 1;
#define VB_CLUSTER(AMN, BMN)                                                                \
  (best_bn == 128 ? launch_gemm<128, AMN, BMN, EPI_STORE>(A, B, lda, ldb, p, stream)         \
                  : launch_gemm<64, AMN, BMN, EPI_STORE>(A, B, lda, ldb, p, stream))
      if (!a_mn && !b_mn) return VB_CLUSTER(false, false);
      if (best_bn == 128) {
        if (!a_mn && b_mn) return launch_gemm<128, false, true, EPI_STORE>(A, B, lda, ldb, p, stream);
        if (a_mn && b_mn) return launch_gemm<128, true, true, EPI_STORE>(A, B, lda, ldb, p, stream);
        return launch_gemm<128, true, false, EPI_STORE>(A, B, lda, ldb, p, stream);
      }
#undef VB_CLUSTER
      p.k_splits = 1;  // 64-wide tiles exist for the K-major layout only: other layouts take the paths below
      p.k_cluster = 0;
    }
  }
  if (ws != nullptr && counters != nullptr && splitk_mode != 0) {
    // Split K when the output tiles alone leave most SMs idle and K is deep enough to cut. 128-wide tiles by
    // default; VERL_B200_SPLITK_BN=256 selects 256-wide ones (fewer re-reads of A, but more slices to reduce).
    static const int force_bn = []() {
      const char* e = getenv("VERL_B200_SPLITK_BN");
      return e ? atoi(e) : 0;
    }();
    const int nm = (M + BM - 1) / BM, nkb = (K + BK - 1) / BK;
    auto plan = [&](int bn, int& splits, int& per) {
      const int tiles = nm * ((N + bn - 1) / bn);
      splits = vb_num_sms() / (tiles > 0 ? tiles : 1);
      if (splits > nkb / 4) splits = nkb / 4;
      if (splits > 16) splits = 16;
      if (splitk_mode > 1) splits = splitk_mode;
      if (splits < 2) { splits = 1; per = nkb; return; }
      per = (nkb + splits - 1) / splits;
      splits = (nkb + per - 1) / per;
    };
    int s256, p256, s128, p128;
    plan(256, s256, p256);
    plan(128, s128, p128);
    int bn_sk = 128;
    if (force_bn == 256 && s256 >= 2) bn_sk = 256;  // measured slower on the 7B decode shapes (more slices to reduce)
    const int splits = bn_sk == 256 ? s256 : s128, per = bn_sk == 256 ? p256 : p128;
    const int nn = (N + bn_sk - 1) / bn_sk;
    if (N > 128 && splits >= 2 && nm * nn * splits <= vb_num_sms() && num_counters >= 2) {
      const long long need = (long long)splits * nm * BM * nn * bn_sk * 4;
      if (need <= ws_bytes) {
        p.k_splits = splits;
        p.kb_per_split = per;
        p.ws = ws;
        p.counters = counters;
#define VB_SPLITK(AMN, BMN)                                                                  \
  (bn_sk == 256 ? launch_gemm<256, AMN, BMN, EPI_STORE>(A, B, lda, ldb, p, stream)             \
                : launch_gemm<128, AMN, BMN, EPI_STORE>(A, B, lda, ldb, p, stream))
        if (!a_mn && !b_mn) return VB_SPLITK(false, false);
        if (!a_mn && b_mn) return VB_SPLITK(false, true);
        if (a_mn && b_mn) return VB_SPLITK(true, true);
        return VB_SPLITK(true, false);
#undef VB_SPLITK
      }
    }
  }
  // Large problems: CTA pairs on 256 x 256 tiles (enough tiles to keep every pair busy for several rounds).
  static const bool pair_enabled = []() {
    const char* e = getenv("VERL_B200_GEMM_PAIR");
    return !(e && e[0] == '0');
  }();
  if (pair_enabled && !p.rs_stage && M >= 512 && N >= 512 && K >= 256 &&
      (long long)((M + 255) / 256) * ((N + 255) / 256) >= vb_num_sms()) {
    int rc;
    if (!a_mn && !b_mn) rc = launch_gemm_pair<false, false>(A, B, lda, ldb, p, stream);
    else if (!a_mn && b_mn) rc = launch_gemm_pair<false, true>(A, B, lda, ldb, p, stream);
    else if (a_mn && b_mn) rc = launch_gemm_pair<true, true>(A, B, lda, ldb, p, stream);
    else rc = launch_gemm_pair<true, false>(A, B, lda, ldb, p, stream);
    if (rc != -7) return rc;  // -7: the device cannot co-schedule the pairs; use the single-CTA kernel
  }
  // Tile width: the widest BN that still yields about one tile per SM. Skinny problems (decode: M <= 128)
  // fall to BN = 64 / 32 so that the weight matrix is streamed by (nearly) all SMs.
  const int num_m = (M + BM - 1) / BM;
  const int want = vb_num_sms() * 4 / 5;
  auto tiles = [&](int bn) { return num_m * ((N + bn - 1) / bn); };
  int bn = 256;
  if (N <= 128 || tiles(256) < want) bn = 128;
  const bool kk = !a_mn && !b_mn;
  if (kk && bn == 128 && tiles(128) < want) bn = 64;
  if (kk && bn == 64 && tiles(64) < want && !p.rs_stage) bn = 32;
  if (N <= 32 && kk) bn = 32;
  else if (N <= 64 && kk) bn = bn < 64 ? bn : 64;
  if (p.rs_stage && bn < 64) p.rs_stage = 0;  // no room for the staging area next to ten pipeline stages
#define VB_DISPATCH(AMN, BMN)                                                              \
  (bn == 256 ? launch_gemm<256, AMN, BMN, EPI_STORE>(A, B, lda, ldb, p, stream)             \
             : launch_gemm<128, AMN, BMN, EPI_STORE>(A, B, lda, ldb, p, stream))
  if (kk) {
    if (bn == 64) return launch_gemm<64, false, false, EPI_STORE>(A, B, lda, ldb, p, stream);
    if (bn == 32) return launch_gemm<32, false, false, EPI_STORE>(A, B, lda, ldb, p, stream);
    return VB_DISPATCH(false, false);
  }
  if (!a_mn && b_mn) return VB_DISPATCH(false, true);
  if (a_mn && b_mn) return VB_DISPATCH(true, true);
  return VB_DISPATCH(true, false);
#undef VB_DISPATCH
}

extern "C" int vb_gemm_bf16_ws(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                               long long lda, long long ldb, long long ldc, int a_mn, int b_mn, int out_fp32,
                               int accumulate, float* ws, long long ws_bytes, int* counters, int num_counters,
                               int* status, cudaStream_t stream) {
  return gemm_bf16_run(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_fp32, accumulate, ws, ws_bytes, counters,
                       num_counters, status, stream, nullptr, 0, 0);
}

// GEMM -> reduce-scatter, first half: C = A [M, K] . B [N, K]^T is this rank's partial sum of a row-parallel linear
// layer. Row r of the result belongs to rank r / rows_per_rank; the epilogue stores every tile straight into
// dsts[owner] (this rank's slot [rows_per_rank, N] in the owner's receive buffer, peer memory), so the transfer
// over NVLink overlaps the tiles still being computed. The owner adds the slots up after a cross-rank barrier
// (vb_peer_sum_slots). Same tiling, split-K and CTA-pair dispatch as the plain GEMM.
extern "C" int vb_gemm_rs_bf16(const void* A, const void* B, const void* bias, int M, int N, int K, long long lda,
                               long long ldb, long long ldc, void* const* dsts, int world, int rows_per_rank,
                               int out_fp32, float* ws, long long ws_bytes, int* counters, int num_counters,
                               int* status, cudaStream_t stream) {
  if (dsts == nullptr) return -3;
  return gemm_bf16_run(A, B, dsts[0], bias, M, N, K, lda, ldb, ldc, 0, 0, out_fp32, 0, ws, ws_bytes, counters,
                       num_counters, status, stream, dsts, world, rows_per_rank);
}

// Grouped GEMM for mixture-of-experts layers, one launch for all experts.
//   mode 1 (forward / input gradients): A [P, K] holds the routed tokens sorted by expert, every expert's rows padded
//     to a multiple of 128; blk_expert[P / 128] names the expert of each 128-row block (< 0: unused block, skipped).
//     b_mn = 0: B = [E, N, K], C[rows of e] = A . B[e]^T;  b_mn = 1: B = [E, K, N], C = A . B[e].
//   mode 2 (weight gradients): A stored [P, M], B stored [P, N] (a_mn = b_mn = 1), C = [E, M, N] fp32,
//     C[e] += A[rows of e]^T . B[rows of e]; expert_off[E + 1] are the padded row offsets (multiples of 128).
// N (K for b_mn) must be a multiple of 64 in mode 1 so that a tile never reads the next expert's matrix into the
// contraction; M, N arbitrary otherwise. Nothing is read back to the host: routing stays on the device.
extern "C" int vb_grouped_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                    long long ldb, long long ldc, int a_mn, int b_mn, int out_fp32, int accumulate,
                                    int mode, int E, const int* blk_expert, const int* expert_off, int* status,
                                    cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || E <= 0) return 0;
  if ((lda & 7) || (ldb & 7)) return -3;
  if (mode == 1 && (a_mn || blk_expert == nullptr || (M % BM) != 0 || ((b_mn ? K : N) % 64) != 0)) return -3;
  if (mode == 2 && (!a_mn || !b_mn || !out_fp32 || !accumulate || expert_off == nullptr)) return -3;
  if (mode != 1 && mode != 2) return -3;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.out_fp32 = out_fp32; p.accumulate = accumulate; p.status = status;
  p.k_splits = 1;
  p.grp_mode = mode; p.grp_E = E; p.grp_blk_expert = blk_expert; p.grp_off = expert_off;
  // the tensor map of B spans all experts: [E * rows, cols]
  GemmParams q = p;
  const bool wide = N >= 512;
  if (mode == 1) {
    // B extents for the descriptor: K-major [E * N, K]; MN-major [E * K, N]
    if (!b_mn) { q.N = E * N; } else { q.K = E * K; }
  }
  CUtensorMap tmA, tmB;
  int rc;
  const int bn = wide ? 256 : 128;
  if (a_mn) rc = vb_make_tmap_2d(&tmA, A, 2, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)lda * 2, 64, BK);
  else rc = vb_make_tmap_2d(&tmA, A, 2, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)lda * 2, BK, BM);
  if (rc) return rc;
  if (b_mn) rc = vb_make_tmap_2d(&tmB, B, 2, (uint64_t)q.N, (uint64_t)q.K, (uint64_t)ldb * 2, 64, BK);
  else rc = vb_make_tmap_2d(&tmB, B, 2, (uint64_t)q.K, (uint64_t)q.N, (uint64_t)ldb * 2, BK, bn);
  if (rc) return rc;
  const int num_m = (M + BM - 1) / BM, num_n = (N + bn - 1) / bn;
  long long units = (long long)num_m * num_n * (mode == 2 ? E : 1);
  if (units <= 0) return 0;
  const int grid = units < vb_num_sms() ? (int)units : vb_num_sms();
#define VB_GRP(BNV, AMN, BMN)                                                                                     \
  do {                                                                                                            \
    auto kern = gemm_kernel<BNV, AMN, BMN, EPI_STORE>;                                                            \
    static bool attr_set = false;                                                                                 \
    if (!attr_set) {                                                                                              \
      VB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout<BNV>::DYN_BYTES)); \
      attr_set = true;                                                                                            \
    }                                                                                                             \
    kern<<<grid, NUM_THREADS, SmemLayout<BNV>::DYN_BYTES, stream>>>(tmA, tmB, p);                                 \
  } while (0)
  if (mode == 2) {
    if (wide) VB_GRP(256, true, true); else VB_GRP(128, true, true);
  } else if (!b_mn) {
    if (wide) VB_GRP(256, false, false); else VB_GRP(128, false, false);
  } else {
    if (wide) VB_GRP(256, false, true); else VB_GRP(128, false, true);
  }
#undef VB_GRP
  vb_count_launch();
  return (int)cudaGetLastError();
}

// Fused all-gather + GEMM: C[M,N] = A . W^T where W [N,K] is not there yet. Every rank holds a contiguous slice
// (`shard_elems` elements) of a flat bf16 vector that contains W at element offset `w_off`; `srcs[r]` is rank r's
// slice (a peer-mapped pointer for remote ranks). While the tensor-core warps run, four copy warps per CTA pull
// W chunk by chunk (in tile order) into `W_full`, and a tile's TMA loads wait only for the chunk they need: the
// NVLink transfer hides under the MMAs of the earlier tiles. `ready` holds ceil(N/256) counters (zeroed here).
// The caller guarantees that every rank's slice is final (a cross-rank barrier after the last update of the
// slices) and that no rank rewrites its slice before all ranks have finished this call.
// w_off, shard_elems and K must be multiples of 8; the kernel is launched cooperatively (its CTAs wait on each
// other's copies, so all of them must be resident).
extern "C" int vb_ag_gemm_bf16(const void* A, void* W_full, void* C, const void* bias, int M, int N, int K,
                               long long lda, long long ldc, const void* const* srcs, int world, long long shard_elems,
                               long long w_off, unsigned* ready, int out_fp32, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (K & 7) || (w_off & 7) || (shard_elems & 7) || world > AG_MAX_RANKS || world < 1) return -3;
  if ((w_off + (long long)N * K + shard_elems - 1) / shard_elems > world) return -3;
  constexpr int BN = 256;
  using L = SmemLayout<BN>;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.out_fp32 = out_fp32; p.status = status;
  p.k_splits = 1;
  for (int r = 0; r < world; ++r) p.ag_src[r] = srcs[r];
  p.ag_shard = shard_elems; p.ag_w_off = w_off;
  p.ag_dst = reinterpret_cast<__nv_bfloat16*>(W_full);
  p.ag_ready = ready;
  CUtensorMap tmA, tmB;
  int rc = vb_make_tmap_2d(&tmA, A, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM);
  if (rc) return rc;
  rc = vb_make_tmap_2d(&tmB, W_full, 2, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, BK, BN);
  if (rc) return rc;
  auto kern = gemm_kernel<BN, false, false, EPI_STORE_AG>;
  static bool attr_set = false;
  if (!attr_set) {
    VB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES));
    attr_set = true;
  }
  const int num_n = (N + BN - 1) / BN;
  const int units = ((M + BM - 1) / BM) * num_n;
  const int grid = units < vb_num_sms() ? units : vb_num_sms();
  VB_CUDA_CHECK(cudaMemsetAsync(ready, 0, sizeof(unsigned) * num_n, stream));
  void* args[] = {(void*)&tmA, (void*)&tmB, (void*)&p};
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)kern, dim3(grid), dim3(NUM_THREADS + AG_COPY_THREADS), args,
                                              L::DYN_BYTES, stream);
  vb_count_launch();
  return (int)e;
}

extern "C" int vb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                            long long lda, long long ldb, long long ldc, int a_mn, int b_mn, int out_fp32,
                            int accumulate, int* status, cudaStream_t stream) {
  return vb_gemm_bf16_ws(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_fp32, accumulate, nullptr, 0, nullptr,
                         0, status, stream);
}

// Number of vocab splits the fused lm_head kernel uses for (T, V); the caller sizes
// the scratch as T * splits * 4 floats.
extern "C" int vb_lmhead_num_splits(int T, int V) {
  const int num_m = (T + BM - 1) / BM;
  const int num_n = (V + 255) / 256;
  int splits = (2 * vb_num_sms() + num_m - 1) / num_m;
  if (splits < 1) splits = 1;
  if (splits > num_n) splits = num_n;
  const int per = (num_n + splits - 1) / splits;
  return (num_n + per - 1) / per;
}

// Fused lm_head forward: logits = hidden . weight^T * inv_temperature are never written.
//   hidden [T,H] bf16, weight [V,H] bf16, labels [T] int64.
//   scratch: T * vb_lmhead_num_splits(T,V) * 4 floats.
//   outputs (fp32, each [T], any may be null): logprob of label, entropy, lse, mean logit under p.
extern "C" int vb_lmhead_logprob_fwd(const void* hidden, const void* weight, const long long* labels, int T, int H,
                                     int V, float inv_temperature, float* scratch, float* logprob, float* entropy,
                                     float* lse, float* mean, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H & 7) return -3;
  GemmParams p{};
  p.M = T; p.N = V; p.K = H;
  p.labels = labels; p.inv_temperature = inv_temperature;
  const int num_n = (V + 255) / 256;
  p.num_splits = vb_lmhead_num_splits(T, V);
  p.nblk_per_split = (num_n + p.num_splits - 1) / p.num_splits;
  p.partials = scratch; p.status = status;
  int rc = launch_gemm<256, false, false, EPI_LSE>(hidden, weight, H, H, p, stream);
  if (rc) return rc;
  lse_merge_kernel<<<(T + 127) / 128, 128, 0, stream>>>(reinterpret_cast<const float4*>(scratch), T, p.num_splits,
                                                        logprob, entropy, lse, mean);
  vb_count_launch();
  return (int)cudaGetLastError();
}

// d_logits chunk for the fused lm_head backward: recomputes logits[T, n_offset : n_offset+Vc]
// and writes d_logits (bf16, [T, ldc]) given per-row lse / mean and upstream gradients.
//   weight_chunk points at weight[n_offset, 0].
extern "C" int vb_lmhead_dlogits(const void* hidden, const void* weight_chunk, const long long* labels, int T, int H,
                                 int Vc, int n_offset, float inv_temperature, const float* lse, const float* mean,
                                 const float* g_logprob, const float* g_entropy, void* dlogits, long long ldc,
                                 int* status, cudaStream_t stream) {
  if (T <= 0 || Vc <= 0) return 0;
  if (H & 7) return -3;
  GemmParams p{};
  p.M = T; p.N = Vc; p.K = H;
  p.C = dlogits; p.ldc = ldc;
  p.labels = labels; p.inv_temperature = inv_temperature;
  p.row_lse = lse; p.row_mean = mean; p.g_logprob = g_logprob; p.g_entropy = g_entropy;
  p.n_offset = n_offset; p.status = status;
  return launch_gemm<256, false, false, EPI_DLOGITS>(hidden, weight_chunk, H, H, p, stream);
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant of the fused lm_head forward (declared in lmhead_static.h).
#include "lmhead_static.h"

#include <cstdio>
#include <mutex>

static __device__ __align__(256) float g_lmhead_static_scratch[VB_LMHEAD_STATIC_SCRATCH_FLOATS];

extern "C" int vb_lmhead_static_scratch_floats(void) { return VB_LMHEAD_STATIC_SCRATCH_FLOATS; }

extern "C" int vb_lmhead_logprob_fwd_static(const void* hidden, const void* weight, const long long* labels, int T,
                                            int H, int V, float inv_temperature, float* logprob, float* entropy,
                                            float* lse, float* mean, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (V <= 0 || H <= 0 || (H & 7)) return -3;
  const long long need = (long long)T * vb_lmhead_num_splits(T, V) * 4;
  if (need > (long long)VB_LMHEAD_STATIC_SCRATCH_FLOATS) {
    fprintf(stderr,
            "vb_lmhead_logprob_fwd_static: T=%d V=%d needs %lld scratch floats, the static array holds %d; "
            "use vb_lmhead_logprob_fwd with caller-provided scratch\n",
            T, V, need, VB_LMHEAD_STATIC_SCRATCH_FLOATS);
    return -4;
  }
  // per-device address of the array, resolved once
  static std::mutex mu;
  static float* scratch_of[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return -5;
  float* ptr = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (scratch_of[dev] == nullptr) {
      float* p = nullptr;
      e = cudaGetSymbolAddress((void**)&p, g_lmhead_static_scratch);
      if (e != cudaSuccess || p == nullptr) {
        fprintf(stderr, "vb_lmhead_logprob_fwd_static: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
        return -5;
      }
      scratch_of[dev] = p;
    }
    ptr = scratch_of[dev];
  }
  return vb_lmhead_logprob_fwd(hidden, weight, labels, T, H, V, inv_temperature, ptr, logprob, entropy, lse, mean,
                               status, stream);
}
