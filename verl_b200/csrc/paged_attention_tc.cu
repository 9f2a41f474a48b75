// Paged-KV decode attention on tcgen05 (head_dim 128, up to 16 query heads per KV head).
//
// One CTA per (sequence, KV head, split). Work is transposed so that all 128 epilogue threads are busy
// although a decode step has only G = Hq/Hk query rows:
//     S^T[keys x heads]  = K_chunk[128 keys x 128 dims] . Q^T          (M = 128 keys,  N = 16 heads, K = 128 dims)
//     O^T[dims x heads] += V_chunk^T[128 dims x 128 keys] . P[keys x heads]  (M = 128 dims, N = 16 heads, K = 128 keys)
// TMEM lane i of S^T is key i of the chunk, lane i of O^T is output dim i: every thread of warps 0..3 owns
// one key during the softmax and one output dimension during accumulation (16 fp32 values each).
//
//   warps 0..3 : softmax over the chunk (max / sum across the 128 key-threads), write P^T (bf16) into shared
//                memory in the 128-byte-swizzled K-major layout, then fold O^T of the chunk into the running
//                output held in registers (flash-decoding rescale)
//   warp 4     : TMA producer: the pages of a chunk are fetched with per-CTA 2-D tiled loads straight from
//                the paged cache ([num_blocks, Hk, block_size, 128]) into a ring of three 32 KB slots that
//                alternates K and V tiles; shared memory stays near 111 KB so that two CTAs share an SM and
//                one CTA's softmax chain overlaps the other's loads and MMAs
//   warp 5     : TMEM allocation + single-thread tcgen05.mma issue
//
// V needs no transpose: [keys, dims] with dims contiguous is exactly an "MN-major" A operand.
// All waits are bounded; on expiry the status word is set and the CTA leaves through its teardown.
#include "common.cuh"
#include <cstdlib>
#include "host_utils.h"

namespace vb {

constexpr int TC_CHUNK = 128;   // keys per chunk
constexpr int TC_D = 128;       // head dim
constexpr int TC_NH = 16;       // padded number of query heads per KV head (UMMA N)
constexpr int TC_STAGES = 3;    // ring slots of one 32 KB tile each; tiles alternate K(0), V(0), K(1), V(1), ...
constexpr int TC_THREADS = 192;
constexpr int KV_TILE_BYTES = TC_CHUNK * TC_D * 2;        // 32 KB (two 64-wide halves of 16 KB)
constexpr int STAGE_BYTES_TC = KV_TILE_BYTES;
constexpr int Q_BYTES = TC_NH * TC_D * 2;                 // 4 KB: two 64-dim k-blocks of 2 KB
constexpr int P_BYTES = TC_NH * TC_CHUNK * 2;             // 4 KB: two 64-key k-blocks of 2 KB
constexpr int TC_BAR_OFF = TC_STAGES * STAGE_BYTES_TC + Q_BYTES + 2 * P_BYTES;
constexpr int TC_BT_OFF = TC_BAR_OFF + 16 * 8 + 64;
constexpr int TC_BT_MAX = 256;  // block-table entries of this CTA's key range staged in shared memory
constexpr int TC_RED_OFF = TC_BT_OFF + TC_BT_MAX * 4;
constexpr int TC_SMEM = TC_RED_OFF + 2 * TC_NH * 4 * 4 + 1024;  // about 111 KB: two CTAs per SM

struct DecodeTcParams {
  const __nv_bfloat16* q;
  long long q_stride;
  const int* block_table;
  int max_blocks;
  const int* seq_lens;
  int Hq, Hk, block_size;
  float scale;
  int num_splits;
  __nv_bfloat16* out;
  long long out_stride;
  float* o_part;
  float* ml_part;
  int* status;
};

// byte offset of element (row r, col k) inside a K-major, 128-byte-swizzled operand of `rows` rows whose
// k extent is split in 64-element blocks of rows*128 bytes
__device__ __forceinline__ uint32_t sw128_off(int r, int k, int rows) {
  const int kb = k >> 6, c16 = (k & 63) >> 3;
  return (uint32_t)(kb * rows * 128 + (r >> 3) * 1024 + (r & 7) * 128 + ((c16 ^ (r & 7)) << 4) + (k & 7) * 2);
}

__device__ __forceinline__ void bar_sync_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// barrier over the 128 softmax threads that also and-reduces a predicate, so that all of them leave the
// chunk loop in the same iteration
__device__ __forceinline__ bool bar_and_128(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.red.and.pred p, 1, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

__global__ void __launch_bounds__(TC_THREADS, 2)
paged_decode_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                       const DecodeTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage0 = smem;
  uint8_t* q_s = smem + TC_STAGES * STAGE_BYTES_TC;
  uint8_t* p_s = q_s + Q_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + TC_BAR_OFF);
  uint64_t* empty = full + TC_STAGES;
  uint64_t* s_full = empty + TC_STAGES;
  uint64_t* p_ready = s_full + 2;
  uint64_t* o_full = p_ready + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* bt_s = reinterpret_cast<int*>(smem + TC_BT_OFF);
  float (*red_s)[4] = reinterpret_cast<float (*)[4]>(smem + TC_RED_OFF);           // per-warp chunk maxima
  float (*red2_s)[4] = reinterpret_cast<float (*)[4]>(smem + TC_RED_OFF + TC_NH * 16);  // per-warp chunk sums

  const int b = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
  const int G = p.Hq / p.Hk;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);
      mbar_init(&o_full[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  // Q^T operand: [16 heads x 128 dims], rows >= G are zero. P buffers start zeroed (rows >= G stay zero).
  for (int i = tid; i < (Q_BYTES + 2 * P_BYTES) / 16; i += TC_THREADS) reinterpret_cast<uint4*>(q_s)[i] = make_uint4(0, 0, 0, 0);
  if (warp == 5) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();  // TMEM is held: a dependent kernel may take what is left
  pdl_wait();     // nothing above reads or writes global memory

  const int seq_len = p.seq_lens[b];
  const int chunks_total = (seq_len + TC_CHUNK - 1) / TC_CHUNK;
  const int per_split = (chunks_total + p.num_splits - 1) / p.num_splits;
  const int c_begin = split * per_split;
  const int c_end = min(chunks_total, c_begin + per_split);
  const int n_chunks = max(c_end - c_begin, 0);
  // block-table entries of this CTA's pages: the producer must not chase global loads between its copies
  const int pages_per_chunk = TC_CHUNK / p.block_size;
  const int n_pages = (seq_len + p.block_size - 1) / p.block_size;
  const int page_base = c_begin * pages_per_chunk;
  {
    const int* bt = p.block_table + (long long)b * p.max_blocks;
    const int cnt = min(min(n_chunks * pages_per_chunk, n_pages - page_base), TC_BT_MAX);
    for (int i = tid; i < cnt; i += TC_THREADS) bt_s[i] = bt[page_base + i];
  }
  for (int i = tid; i < G * TC_D; i += TC_THREADS) {
    const int g = i / TC_D, d = i % TC_D;
    const __nv_bfloat16 v = p.q[(long long)b * p.q_stride + (long long)(h * G + g) * TC_D + d];
    *reinterpret_cast<__nv_bfloat16*>(q_s + sw128_off(g, d, TC_NH)) = v;
  }
  fence_proxy_async_smem();
  __syncthreads();

  if (warp == 4) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0 && n_chunks > 0) {
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      const int* bt = p.block_table + (long long)b * p.max_blocks;
      for (int t = 0; t < 2 * n_chunks; ++t) {
        const int s = t % TC_STAGES;
        const uint32_t par = ((t / TC_STAGES) & 1) ^ 1;
        if (*abort_flag || !mbar_wait(&empty[s], par)) {
          report_error(p.status, ERR_WAIT_EMPTY, t);
          *abort_flag = 1;
          break;
        }
        mbar_arrive_expect_tx(&full[s], STAGE_BYTES_TC);
        uint8_t* dst = stage0 + s * STAGE_BYTES_TC;
        const CUtensorMap* tm = (t & 1) ? &tmV : &tmK;
        const int page0 = (c_begin + (t >> 1)) * pages_per_chunk;
        for (int pg = 0; pg < pages_per_chunk; ++pg) {
          // pages past the end of the sequence re-read the sequence's last page: finite data, masked later
          const int pi = min(page0 + pg, n_pages - 1);
          const int rel = pi - page_base;
          const int blk = rel < TC_BT_MAX ? bt_s[rel] : bt[pi];
          const int row = (blk * p.Hk + h) * p.block_size;
          const int off = pg * p.block_size * 128;
          tma_load_2d(dst + off, tm, &full[s], 0, row);
          tma_load_2d(dst + 16384 + off, tm, &full[s], 64, row);
        }
      }
    }
  } else if (warp == 5) {
    // -------------------------------- MMA issuer --------------------------------
    if (lane == 0 && n_chunks > 0) {
      constexpr uint32_t idesc_qk = umma_idesc(1, 1, 0, 0, 128, TC_NH);  // A = K (K-major), B = Q^T (K-major)
      constexpr uint32_t idesc_pv = umma_idesc(1, 1, 1, 0, 128, TC_NH);  // A = V (MN-major), B = P^T (K-major)
      const uint32_t q_addr = smem_u32(q_s);
      bool ok = true;
      auto issue_qk = [&](int c) -> bool {
        const int t = 2 * c, s = t % TC_STAGES;
        if (*abort_flag || !mbar_wait(&full[s], (t / TC_STAGES) & 1)) {
          report_error(p.status, ERR_WAIT_FULL, t);
          *abort_flag = 1;
          return false;
        }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(stage0 + s * STAGE_BYTES_TC);
        const uint32_t d_tmem = tmem_base + (c & 1) * TC_NH;
#pragma unroll
        for (int k = 0; k < TC_D / 16; ++k) {
          const uint64_t a = umma_smem_desc(k_addr + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
          const uint64_t bq = umma_smem_desc(q_addr + (k >> 2) * (TC_NH * 128) + (k & 3) * 32, 16, 1024);
          tc_mma_f16(d_tmem, a, bq, idesc_qk, k != 0);
        }
        tc_commit(&s_full[c & 1]);
        tc_commit(&empty[s]);
        return true;
      };
      ok = issue_qk(0);
      for (int c = 0; ok && c < n_chunks; ++c) {
        if (c + 1 < n_chunks) ok = issue_qk(c + 1);
        if (!ok) break;
        const int t = 2 * c + 1, s = t % TC_STAGES;
        if (*abort_flag || !mbar_wait(&full[s], (t / TC_STAGES) & 1)) {
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
        const uint32_t v_addr = smem_u32(stage0 + s * STAGE_BYTES_TC);
        const uint32_t p_addr = smem_u32(p_s + (c & 1) * P_BYTES);
        const uint32_t d_tmem = tmem_base + 32 + (c & 1) * TC_NH;
#pragma unroll
        for (int k = 0; k < TC_CHUNK / 16; ++k) {
          // A: dims are the M side (two 64-dim halves 16 KB apart), 16 keys per step = 16 rows of 128 bytes
          const uint64_t a = umma_smem_desc(v_addr + k * 2048, 16384, 1024);
          const uint64_t bp = umma_smem_desc(p_addr + (k >> 2) * (TC_NH * 128) + (k & 3) * 32, 16, 1024);
          tc_mma_f16(d_tmem, a, bp, idesc_pv, k != 0);
        }
        tc_commit(&o_full[c & 1]);
        tc_commit(&empty[s]);
      }
    }
  } else {
    // ----------------------- softmax + accumulation (128 threads) -----------------------
    float m_run[TC_NH], l_run[TC_NH], o_acc[TC_NH];
#pragma unroll
    for (int g = 0; g < TC_NH; ++g) {
      m_run[g] = -INFINITY;
      l_run[g] = 0.f;
      o_acc[g] = 0.f;
    }
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    bool ok = true;
    float alpha_cur[TC_NH], alpha_nxt[TC_NH];
    // softmax of chunk c: S^T -> P^T (bf16, shared memory), running max / sum, rescale factor of this chunk
    auto softmax_chunk = [&](int c, float (&alpha)[TC_NH]) {
      const int i = c & 1;
      if (*abort_flag || !mbar_wait(&s_full[i], (c >> 1) & 1)) {
        report_error(p.status, ERR_WAIT_TMEM_FULL, c);
        *abort_flag = 1;
        ok = false;
      }
      // every thread of the 4 warps must reach the named barriers: on failure fall through with zeros
      uint32_t sr[16];
      if (ok) {
        tc_fence_after();
        tmem_ld_32x16(tmem_base + lane_base + i * TC_NH, sr);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int g = 0; g < 16; ++g) sr[g] = 0;
      }
      const int key = (c_begin + c) * TC_CHUNK + tid;
      const bool valid = key < seq_len;
      float sc[TC_NH];
#pragma unroll
      for (int g = 0; g < TC_NH; ++g) {
        sc[g] = valid ? __uint_as_float(sr[g]) * p.scale : -INFINITY;
        if (g < G) {
          const float wm = warp_reduce_max(sc[g]);
          if (lane == 0) red_s[g][warp] = wm;
        }
      }
      bar_sync_128();
      uint8_t* pbuf = p_s + i * P_BYTES;
#pragma unroll
      for (int g = 0; g < TC_NH; ++g) {
        alpha[g] = 1.f;
        if (g < G) {
          const float cm = fmaxf(fmaxf(red_s[g][0], red_s[g][1]), fmaxf(red_s[g][2], red_s[g][3]));
          const float nm = fmaxf(m_run[g], cm);
          alpha[g] = __expf(m_run[g] - nm);
          const float pv = valid ? __expf(sc[g] - nm) : 0.f;
          m_run[g] = nm;
          // P^T[g][key] in bf16, swizzled K-major (row = head, k = key within the chunk)
          *reinterpret_cast<__nv_bfloat16*>(pbuf + sw128_off(g, tid, TC_NH)) = __float2bfloat16(pv);
          const float ws = warp_reduce_sum(pv);
          if (lane == 0) red2_s[g][warp] = ws;
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[i]);
      bar_sync_128();
#pragma unroll
      for (int g = 0; g < TC_NH; ++g)
        if (g < G) l_run[g] = l_run[g] * alpha[g] + red2_s[g][0] + red2_s[g][1] + red2_s[g][2] + red2_s[g][3];
    };
    if (n_chunks > 0) {
      softmax_chunk(0, alpha_cur);
      ok = bar_and_128(ok);  // all 128 threads enter (or skip) the loop together
    }
    for (int c = 0; ok && c < n_chunks; ++c) {
      const int i = c & 1;
      // the next chunk's softmax runs while the tensor core works on P.V of this one
      if (c + 1 < n_chunks) softmax_chunk(c + 1, alpha_nxt);
      // O^T of this chunk: lane = output dim
      if (ok && (*abort_flag || !mbar_wait(&o_full[i], (c >> 1) & 1))) {
        report_error(p.status, ERR_WAIT_TMEM_FULL, 1000 + c);
        *abort_flag = 1;
        ok = false;
      }
      if (ok) {
        tc_fence_after();
        uint32_t orr[16];
        tmem_ld_32x16(tmem_base + lane_base + 32 + i * TC_NH, orr);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < TC_NH; ++g)
          if (g < G) o_acc[g] = o_acc[g] * alpha_cur[g] + __uint_as_float(orr[g]);
      }
#pragma unroll
      for (int g = 0; g < TC_NH; ++g) alpha_cur[g] = alpha_nxt[g];
      ok = bar_and_128(ok);  // one failed wait ends the loop for all
    }
    if (ok) {
      const int d = tid;
#pragma unroll
      for (int g = 0; g < TC_NH; ++g) {
        if (g < G) {
          const int hq = h * G + g;
          if (p.num_splits == 1) {
            p.out[(long long)b * p.out_stride + (long long)hq * TC_D + d] =
                __float2bfloat16(l_run[g] > 0.f ? o_acc[g] / l_run[g] : 0.f);
          } else {
            const long long base = ((long long)b * p.Hq + hq) * p.num_splits + split;
            p.o_part[base * TC_D + d] = o_acc[g];
            if (d == 0) {
              p.ml_part[base * 2] = m_run[g];
              p.ml_part[base * 2 + 1] = l_run[g];
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
    tmem_dealloc(tmem_base, 64);
  }
}


// ---------------------------------------------------------------------------------------------------------------
// Persistent variant: the grid is two CTAs per SM, CTA i works on items i, i + grid, i + 2 * grid, ... where an item is
// one (sequence, KV head, split). The per-CTA set-up (barriers, TMEM, zeroed operand rows) is paid once, and the
// producer warp runs ahead into the next item (its Q rows, block-table entries and first K / V tiles) while the
// softmax warps still finish the current one, so the pipeline does not drain between items. Ring stages, S / P / O
// buffers and Q buffers alternate by running counters that continue across items.
// One Q^T operand (a second one would push the CTA over half an SM's shared memory and halve the occupancy): the
// producer refills it as soon as the last QK MMA of the previous item has completed, which the look-ahead issue makes
// early (before that item's last softmax and P.V).
constexpr int TCP_BAR_OFF = TC_STAGES * STAGE_BYTES_TC + Q_BYTES + 2 * P_BYTES;
static_assert(2 * (TCP_BAR_OFF + 20 * 8 + 64 + TC_BT_MAX * 4 + 2 * TC_NH * 4 * 4 + 1024) <= 227 * 1024,
              "two CTAs of the persistent decode kernel must fit in one SM");
constexpr int TCP_BT_OFF = TCP_BAR_OFF + 20 * 8 + 64;
constexpr int TCP_RED_OFF = TCP_BT_OFF + TC_BT_MAX * 4;
constexpr int TCP_SMEM = TCP_RED_OFF + 2 * TC_NH * 4 * 4 + 1024;

struct TcItem {
  int b, h, split, seq_len, c_begin, n_chunks;
};
__device__ __forceinline__ TcItem tc_item(const DecodeTcParams& p, int item) {
  TcItem it;
  it.split = item % p.num_splits;
  const int bh = item / p.num_splits;
  it.h = bh % p.Hk;
  it.b = bh / p.Hk;
  it.seq_len = p.seq_lens[it.b];
  const int chunks_total = (it.seq_len + TC_CHUNK - 1) / TC_CHUNK;
  const int per_split = (chunks_total + p.num_splits - 1) / p.num_splits;
  it.c_begin = it.split * per_split;
  it.n_chunks = max(min(chunks_total, it.c_begin + per_split) - it.c_begin, 0);
  return it;
}

__global__ void __launch_bounds__(TC_THREADS, 2)
paged_decode_tc_persist_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                               const DecodeTcParams p, const int num_items) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage0 = smem;
  uint8_t* q_s = smem + TC_STAGES * STAGE_BYTES_TC;
  uint8_t* p_s = q_s + Q_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + TCP_BAR_OFF);
  uint64_t* empty = full + TC_STAGES;
  uint64_t* s_full = empty + TC_STAGES;
  uint64_t* p_ready = s_full + 2;
  uint64_t* o_full = p_ready + 2;
  uint64_t* q_full = o_full + 2;
  uint64_t* q_empty = q_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* bt_s = reinterpret_cast<int*>(smem + TCP_BT_OFF);  // used by the producer warp only
  float (*red_s)[4] = reinterpret_cast<float (*)[4]>(smem + TCP_RED_OFF);
  float (*red2_s)[4] = reinterpret_cast<float (*)[4]>(smem + TCP_RED_OFF + TC_NH * 16);

  const int G = p.Hq / p.Hk;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pages_per_chunk = TC_CHUNK / p.block_size;

  if (tid == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);
      mbar_init(&o_full[i], 1);
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  // rows >= G of the Q^T operand and of both P buffers stay zero for the whole kernel
  for (int i = tid; i < (Q_BYTES + 2 * P_BYTES) / 16; i += TC_THREADS) reinterpret_cast<uint4*>(q_s)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  if (warp == 5) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();  // TMEM is held: a dependent kernel may take what is left
  pdl_wait();     // nothing above reads or writes global memory

  if (warp == 4) {
    // ------------------- producer: Q rows, block table, K / V tiles of item after item -------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
    }
    uint32_t tg = 0, ig = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
      const TcItem it = tc_item(p, item);
      if (it.n_chunks <= 0) continue;
      const int qb = 0;
      // the Q operand is free once the QK MMAs of the previous item have completed
      int good = 1;  // lane 0 decides for the warp: the lanes must leave the loop together
      if (lane == 0) {
        good = (!*abort_flag && mbar_wait(&q_empty[qb], (ig & 1) ^ 1)) ? 1 : 0;
        if (!good) {
          report_error(p.status, ERR_WAIT_EMPTY, 5000 + item);
          *abort_flag = 1;
        }
      }
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) break;
      {
        const __nv_bfloat16* qrow = p.q + (long long)it.b * p.q_stride + (long long)it.h * G * TC_D;
        uint8_t* qdst = q_s + qb * Q_BYTES;
        for (int idx = lane; idx < G * (TC_D / 8); idx += 32) {
          const int g = idx / (TC_D / 8), c8 = idx % (TC_D / 8);
          const uint4 v = *reinterpret_cast<const uint4*>(qrow + g * TC_D + c8 * 8);
          *reinterpret_cast<uint4*>(qdst + sw128_off(g, c8 * 8, TC_NH)) = v;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&q_full[qb]);
      }
      const int n_pages = (it.seq_len + p.block_size - 1) / p.block_size;
      const int page_base = it.c_begin * pages_per_chunk;
      const int* bt = p.block_table + (long long)it.b * p.max_blocks;
      const int cnt = min(min(it.n_chunks * pages_per_chunk, n_pages - page_base), TC_BT_MAX);
      __syncwarp();
      for (int i = lane; i < cnt; i += 32) bt_s[i] = bt[page_base + i];
      __syncwarp();
      if (lane == 0) {
        for (int t = 0; t < 2 * it.n_chunks; ++t, ++tg) {
          const int s = tg % TC_STAGES;
          const uint32_t par = ((tg / TC_STAGES) & 1) ^ 1;
          if (*abort_flag || !mbar_wait(&empty[s], par)) {
            report_error(p.status, ERR_WAIT_EMPTY, t);
            *abort_flag = 1;
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full[s], STAGE_BYTES_TC);
          uint8_t* dst = stage0 + s * STAGE_BYTES_TC;
          const CUtensorMap* tm = (t & 1) ? &tmV : &tmK;
          const int page0 = (it.c_begin + (t >> 1)) * pages_per_chunk;
          for (int pg = 0; pg < pages_per_chunk; ++pg) {
            const int pi = min(page0 + pg, n_pages - 1);
            const int rel = pi - page_base;
            const int blk = rel < TC_BT_MAX ? bt_s[rel] : bt[pi];
            const int row = (blk * p.Hk + it.h) * p.block_size;
            const int off = pg * p.block_size * 128;
            tma_load_2d(dst + off, tm, &full[s], 0, row);
            tma_load_2d(dst + 16384 + off, tm, &full[s], 64, row);
          }
        }
      }
      tg = __shfl_sync(0xffffffffu, tg, 0);
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
      ++ig;
    }
  } else if (warp == 5) {
    // -------------------------------- MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(1, 1, 0, 0, 128, TC_NH);
      constexpr uint32_t idesc_pv = umma_idesc(1, 1, 1, 0, 128, TC_NH);
      uint32_t tg = 0, cg = 0, ig = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
        const TcItem it = tc_item(p, item);
        if (it.n_chunks <= 0) continue;
        const int qb = 0;
        if (*abort_flag || !mbar_wait(&q_full[qb], ig & 1)) {
          report_error(p.status, ERR_WAIT_FULL, 5000 + item);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t q_addr = smem_u32(q_s + qb * Q_BYTES);
        // tiles of this item: K(c) = tg0 + 2c, V(c) = tg0 + 2c + 1; chunk c uses S / P / O buffer (cg0 + c) & 1
        const uint32_t tg0 = tg, cg0 = cg;
        auto issue_qk = [&](int c) -> bool {
          const uint32_t t = tg0 + 2 * c, s = t % TC_STAGES, cc = cg0 + c;
          if (*abort_flag || !mbar_wait(&full[s], (t / TC_STAGES) & 1)) {
            report_error(p.status, ERR_WAIT_FULL, (int)t);
            *abort_flag = 1;
            return false;
          }
          tc_fence_after();
          const uint32_t k_addr = smem_u32(stage0 + s * STAGE_BYTES_TC);
          const uint32_t d_tmem = tmem_base + (cc & 1) * TC_NH;
#pragma unroll
          for (int k = 0; k < TC_D / 16; ++k) {
            const uint64_t a = umma_smem_desc(k_addr + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
            const uint64_t bq = umma_smem_desc(q_addr + (k >> 2) * (TC_NH * 128) + (k & 3) * 32, 16, 1024);
            tc_mma_f16(d_tmem, a, bq, idesc_qk, k != 0);
          }
          tc_commit(&s_full[cc & 1]);
          tc_commit(&empty[s]);
          if (c == it.n_chunks - 1) tc_commit(&q_empty[qb]);  // the item's last read of its Q operand
          return true;
        };
        ok = issue_qk(0);
        for (int c = 0; ok && c < it.n_chunks; ++c) {
          if (c + 1 < it.n_chunks) ok = issue_qk(c + 1);
          if (!ok) break;
          const uint32_t t = tg0 + 2 * c + 1, s = t % TC_STAGES, cc = cg0 + c;
          if (*abort_flag || !mbar_wait(&full[s], (t / TC_STAGES) & 1)) {
            report_error(p.status, ERR_WAIT_FULL, (int)t);
            *abort_flag = 1;
            ok = false;
            break;
          }
          if (*abort_flag || !mbar_wait(&p_ready[cc & 1], (cc >> 1) & 1)) {
            report_error(p.status, ERR_WAIT_TMEM_EMPTY, (int)cc);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t v_addr = smem_u32(stage0 + s * STAGE_BYTES_TC);
          const uint32_t p_addr = smem_u32(p_s + (cc & 1) * P_BYTES);
          const uint32_t d_tmem = tmem_base + 32 + (cc & 1) * TC_NH;
#pragma unroll
          for (int k = 0; k < TC_CHUNK / 16; ++k) {
            const uint64_t a = umma_smem_desc(v_addr + k * 2048, 16384, 1024);
            const uint64_t bp = umma_smem_desc(p_addr + (k >> 2) * (TC_NH * 128) + (k & 3) * 32, 16, 1024);
            tc_mma_f16(d_tmem, a, bp, idesc_pv, k != 0);
          }
          tc_commit(&o_full[cc & 1]);
          tc_commit(&empty[s]);
        }
        tg += 2 * it.n_chunks;
        cg += it.n_chunks;
        ++ig;
      }
    }
  } else {
    // ----------------------- softmax + accumulation (128 threads) -----------------------
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    bool ok = true;
    uint32_t cg = 0;
    for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
      const TcItem it = tc_item(p, item);
      float m_run[TC_NH], l_run[TC_NH], o_acc[TC_NH];
#pragma unroll
      for (int g = 0; g < TC_NH; ++g) {
        m_run[g] = -INFINITY;
        l_run[g] = 0.f;
        o_acc[g] = 0.f;
      }
      float alpha_cur[TC_NH], alpha_nxt[TC_NH];
      const uint32_t cg0 = cg;
      auto softmax_chunk = [&](int c, float (&alpha)[TC_NH]) {
        const uint32_t cc = cg0 + c;
        const int i = cc & 1;
        if (*abort_flag || !mbar_wait(&s_full[i], (cc >> 1) & 1)) {
          report_error(p.status, ERR_WAIT_TMEM_FULL, (int)cc);
          *abort_flag = 1;
          ok = false;
        }
        uint32_t sr[16];
        if (ok) {
          tc_fence_after();
          tmem_ld_32x16(tmem_base + lane_base + i * TC_NH, sr);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int g = 0; g < 16; ++g) sr[g] = 0;
        }
        const int key = (it.c_begin + c) * TC_CHUNK + tid;
        const bool valid = key < it.seq_len;
        float sc[TC_NH];
#pragma unroll
        for (int g = 0; g < TC_NH; ++g) {
          sc[g] = valid ? __uint_as_float(sr[g]) * p.scale : -INFINITY;
          if (g < G) {
            const float wm = warp_reduce_max(sc[g]);
            if (lane == 0) red_s[g][warp] = wm;
          }
        }
        bar_sync_128();
        uint8_t* pbuf = p_s + i * P_BYTES;
#pragma unroll
        for (int g = 0; g < TC_NH; ++g) {
          alpha[g] = 1.f;
          if (g < G) {
            const float cm = fmaxf(fmaxf(red_s[g][0], red_s[g][1]), fmaxf(red_s[g][2], red_s[g][3]));
            const float nm = fmaxf(m_run[g], cm);
            alpha[g] = __expf(m_run[g] - nm);
            const float pv = valid ? __expf(sc[g] - nm) : 0.f;
            m_run[g] = nm;
            *reinterpret_cast<__nv_bfloat16*>(pbuf + sw128_off(g, tid, TC_NH)) = __float2bfloat16(pv);
            const float ws = warp_reduce_sum(pv);
            if (lane == 0) red2_s[g][warp] = ws;
          }
        }
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[i]);
        bar_sync_128();
#pragma unroll
        for (int g = 0; g < TC_NH; ++g)
          if (g < G) l_run[g] = l_run[g] * alpha[g] + red2_s[g][0] + red2_s[g][1] + red2_s[g][2] + red2_s[g][3];
      };
      if (it.n_chunks > 0) {
        softmax_chunk(0, alpha_cur);
        ok = bar_and_128(ok);
      }
      for (int c = 0; ok && c < it.n_chunks; ++c) {
        const uint32_t cc = cg0 + c;
        const int i = cc & 1;
        if (c + 1 < it.n_chunks) softmax_chunk(c + 1, alpha_nxt);
        if (ok && (*abort_flag || !mbar_wait(&o_full[i], (cc >> 1) & 1))) {
          report_error(p.status, ERR_WAIT_TMEM_FULL, 1000 + (int)cc);
          *abort_flag = 1;
          ok = false;
        }
        if (ok) {
          tc_fence_after();
          uint32_t orr[16];
          tmem_ld_32x16(tmem_base + lane_base + 32 + i * TC_NH, orr);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < TC_NH; ++g)
            if (g < G) o_acc[g] = o_acc[g] * alpha_cur[g] + __uint_as_float(orr[g]);
        }
#pragma unroll
        for (int g = 0; g < TC_NH; ++g) alpha_cur[g] = alpha_nxt[g];
        ok = bar_and_128(ok);
      }
      cg += it.n_chunks;
      if (ok) {
        const int d = tid;
#pragma unroll
        for (int g = 0; g < TC_NH; ++g) {
          if (g < G) {
            const int hq = it.h * G + g;
            if (p.num_splits == 1) {
              p.out[(long long)it.b * p.out_stride + (long long)hq * TC_D + d] =
                  __float2bfloat16(l_run[g] > 0.f ? o_acc[g] / l_run[g] : 0.f);
            } else {
              const long long base = ((long long)it.b * p.Hq + hq) * p.num_splits + it.split;
              p.o_part[base * TC_D + d] = o_acc[g];
              if (d == 0) {
                p.ml_part[base * 2] = m_run[g];
                p.ml_part[base * 2 + 1] = l_run[g];
              }
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
    tmem_dealloc(tmem_base, 64);
  }
}

}  // namespace vb

using namespace vb;

// Returns 1 if the tensor-core decode kernel supports this configuration.
extern "C" int vb_paged_decode_tc_supported(int Hq, int Hk, int D, int block_size) {
  return (D == TC_D && Hk > 0 && Hq % Hk == 0 && Hq / Hk <= TC_NH && block_size >= 8 && block_size <= 128 &&
          TC_CHUNK % block_size == 0)
             ? 1
             : 0;
}

int vb_decode_merge_128(const float* o_part, const float* ml_part, int B, int Hq, int num_splits, void* out,
                        long long out_stride, cudaStream_t stream);

// Same contract as vb_paged_decode (caches [NB, Hk, block_size, 128] bf16, partial results merged here);
// num_blocks is needed to describe the cache to TMA, status receives the code of a wait that ran out.
extern "C" int vb_paged_decode_tc(const void* q, long long q_stride, const void* kc, const void* vc, int num_blocks,
                                  const int* block_table, int max_blocks, const int* seq_lens, int B, int Hq, int Hk,
                                  int block_size, float scale, int num_splits, void* out, long long out_stride,
                                  float* work, int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (!vb_paged_decode_tc_supported(Hq, Hk, TC_D, block_size)) return -3;
  CUtensorMap tmK, tmV;
  const uint64_t rows = (uint64_t)num_blocks * Hk * block_size;
  int rc = vb_make_tmap_2d(&tmK, kc, 2, TC_D, rows, TC_D * 2, 64, block_size);
  if (rc) return rc;
  rc = vb_make_tmap_2d(&tmV, vc, 2, TC_D, rows, TC_D * 2, 64, block_size);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    VB_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM));
    attr_set = true;
  }
  DecodeTcParams p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_stride;
  p.block_table = block_table;
  p.max_blocks = max_blocks;
  p.seq_lens = seq_lens;
  p.Hq = Hq; p.Hk = Hk; p.block_size = block_size;
  p.scale = scale;
  p.num_splits = num_splits;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.out_stride = out_stride;
  p.o_part = work;
  p.ml_part = work ? work + (long long)B * Hq * num_splits * TC_D : nullptr;
  p.status = status;
  static const bool persist = []() {
    const char* e = getenv("VERL_B200_DECODE_PERSIST");  // 0 = one CTA per (sequence, head, split)
    return !(e && e[0] == '0');
  }();
  const int items = B * Hk * num_splits;
  // the persistent kernel loads Q rows with 16-byte loads and pays off when CTAs get more than one item
  if (persist && items > 2 * vb_num_sms() && (q_stride & 7) == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0) {
    static bool attr2_set = false;
    if (!attr2_set) {
      VB_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_tc_persist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         TCP_SMEM));
      attr2_set = true;
    }
    rc = (int)vb_launch_pdl(paged_decode_tc_persist_kernel, dim3(2 * vb_num_sms()), dim3(TC_THREADS), TCP_SMEM, stream,
                            1, tmK, tmV, p, items);
  } else {
    dim3 grid(B, Hk, num_splits);
    rc = (int)vb_launch_pdl(paged_decode_tc_kernel, grid, dim3(TC_THREADS), TC_SMEM, stream, 1, tmK, tmV, p);
  }
  vb_count_launch(num_splits > 1 ? 2 : 1);
  if (rc == 0) rc = (int)cudaGetLastError();
  if (rc || num_splits == 1) return rc;
  return vb_decode_merge_128(p.o_part, p.ml_part, B, Hq, num_splits, out, out_stride, stream);
}
