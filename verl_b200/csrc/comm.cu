// Collectives over NVLink peer memory, written as kernels (no NCCL on these paths).
//
// Every rank maps every peer's symmetric buffers (allocation and handle exchange are done by the
// host through torch's symmetric-memory allocator); kernels then read peers with plain ld.global
// over NVLink or, where a multicast mapping exists, with multimem.ld_reduce through NVSwitch.
// No TMA is issued on peer memory and no cluster-wide broadcast loads are used anywhere.
//
// Synchronisation: one signal pad per rank, `world` 32-bit slots per channel. A barrier writes a
// monotonically increasing epoch into slot [my rank] of every peer's pad and waits until all slots
// of its own pad reach the epoch. Waits are bounded (VB_WAIT_LIMIT_NS): on expiry the kernel
// records ERR_WAIT_FLAG in the status word and returns, so a missing peer never hangs the GPU.
//
// Kernels:
//   peer_barrier            all ranks arrive / depart (also orders prior writes: release/acquire at system scope)
//   peer_all_gather         out[p*shard : (p+1)*shard] = peer p's shard (replaces NCCL all-gather in ZeRO-3)
//   peer_reduce_scatter_add dst[i] += scale * sum_p peer p's full[rank*shard + i]  (fp32; grad reduce-scatter
//                           fused with the scale and the accumulation into the optimizer's gradient shard)
//   nvls_reduce_scatter_add same through multimem.ld_reduce (in-switch add)
//   peer_sum_slots          second half of GEMM -> reduce-scatter: the GEMM epilogues of all ranks have stored their
//                           partial rows into this rank's receive slots; barrier, then sum the slots locally
//   moe_dispatch / combine  expert-parallel MoE: tokens pushed into the expert owner's grouped-GEMM-ready receive
//                           buffer; expert outputs pulled back and mixed with the routing weights
//   tp_allreduce_rmsnorm    tensor-parallel row-parallel epilogue: all-reduce of the ranks' partial products fused with
//                           the residual add and the RMSNorm of the next block; device-side epoch (graph-replayable)
//   peer_a2a_chunks         all-to-all of row chunks (Ulysses: gather the sequence / scatter the heads and back), pulled
//                           straight into the destination layout
//   peer_segment_copy       table-driven gather of byte ranges from peers into a local buffer: the
//                           train -> rollout weight reshard (FSDP shards -> TP/EP layout) in one launch
#include "common.cuh"
#include "host_utils.h"

namespace vb {

constexpr int MAX_RANKS = 16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Block 0 performs the cross-rank handshake; the other blocks of the grid are released through a
// local flag in global memory (grid-local, same bounded wait).
__device__ bool barrier_all_ranks(const PeerPtrs& pads, int rank, int world, int channel, uint32_t epoch,
                                  int* status) {
  // each thread t < world handles peer t
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  __threadfence_system();
  if ((int)threadIdx.x < world) {
    uint32_t* remote = reinterpret_cast<uint32_t*>(pads.p[threadIdx.x]) + channel * MAX_RANKS + rank;
    st_release_sys(remote, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(pads.p[rank]) + channel * MAX_RANKS + threadIdx.x;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    // epochs only grow; signed difference tolerates wrap-around
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > VB_WAIT_LIMIT_NS) {
        report_error(status, ERR_WAIT_FLAG, (int)threadIdx.x);
        ok_s = 0;
        break;
      }
    }
  }
  __syncthreads();
  return ok_s != 0;
}

__global__ void peer_barrier_kernel(PeerPtrs pads, int rank, int world, int channel, uint32_t epoch, int* status) {
  vb_jitter(1u);
  barrier_all_ranks(pads, rank, world, channel, epoch, status);
}

// grid-wide: block 0 does the handshake, then publishes `epoch` in *gate; other blocks wait on *gate.
__device__ bool grid_enter(const PeerPtrs& pads, int rank, int world, int channel, uint32_t epoch, uint32_t* gate,
                           int* status) {
  __shared__ int ok_b;
  if (blockIdx.x == 0) {
    bool ok = barrier_all_ranks(pads, rank, world, channel, epoch, status);
    if (threadIdx.x == 0) {
      st_release_sys(gate, ok ? epoch : (epoch | 0x80000000u));
      ok_b = ok ? 1 : 0;
    }
  } else if (threadIdx.x == 0) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0, v;
    ok_b = 1;
    while (((v = ld_acquire_sys(gate)) & 0x7fffffffu) != (epoch & 0x7fffffffu)) {
      if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > 2 * VB_WAIT_LIMIT_NS) {
        report_error(status, ERR_WAIT_FLAG, 1000 + (int)blockIdx.x);
        ok_b = 0;
        break;
      }
    }
    if (ok_b && (v & 0x80000000u)) ok_b = 0;
  }
  __syncthreads();
  return ok_b != 0;
}

// out (local) <- all peers' shards. srcs.p[r] = base of rank r's symmetric buffer; the shard sits at byte
// offset src_off in every rank's buffer. Units of 16 bytes.
__global__ void peer_all_gather_kernel(PeerPtrs srcs, PeerPtrs pads, long long src_off16, uint4* __restrict__ out,
                                       long long shard16, int rank, int world, int channel, uint32_t epoch,
                                       uint32_t* gate, int* status) {
  vb_jitter(2u);
  if (!grid_enter(pads, rank, world, channel, epoch, gate, status)) return;
  const long long total = shard16 * world;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += stride) {
    // start each rank on a different peer so the links are used evenly
    const long long j = (i + (long long)rank * shard16) % total;
    const int p = (int)(j / shard16);
    const long long k = j - (long long)p * shard16;
    const uint4* src = reinterpret_cast<const uint4*>(srcs.p[p]) + src_off16 + k;
    out[j] = *src;
  }
}

// dst[i] += scale * sum_p full_p[rank*shard + i], i in [0, shard). fulls.p[r] = base of rank r's symmetric
// gradient buffer (the unit's full gradient at float offset full_off). float4 granularity. The loads of all
// W peers (W = world size, compile time) are issued before the first add, so that one NVLink round trip covers
// W * U * 16 bytes per thread.
template <int W, int U>
__global__ void peer_reduce_scatter_add_kernel(PeerPtrs fulls, PeerPtrs pads, long long full_off4,
                                               float4* __restrict__ dst, long long shard4, float scale, int rank,
                                               int world, int channel, uint32_t epoch, uint32_t* gate, int* status) {
  vb_jitter(3u);
  if (!grid_enter(pads, rank, world, channel, epoch, gate, status)) return;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long base = full_off4 + (long long)rank * shard4;
  const float4* src[W];
#pragma unroll
  for (int q = 0; q < W; ++q) src[q] = reinterpret_cast<const float4*>(fulls.p[(rank + q) % W]) + base;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < shard4; i0 += stride * U) {
    float4 v[W][U];
#pragma unroll
    for (int q = 0; q < W; ++q) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        v[q][u] = i < shard4 ? src[q][i] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < shard4) {
        float4 acc = v[0][u];
#pragma unroll
        for (int q = 1; q < W; ++q) {
          acc.x += v[q][u].x; acc.y += v[q][u].y; acc.z += v[q][u].z; acc.w += v[q][u].w;
        }
        float4 d = dst[i];
        d.x += scale * acc.x; d.y += scale * acc.y; d.z += scale * acc.z; d.w += scale * acc.w;
        dst[i] = d;
      }
    }
  }
}

// any world size (peers visited one after the other)
__global__ void peer_reduce_scatter_add_generic_kernel(PeerPtrs fulls, PeerPtrs pads, long long full_off4,
                                                       float4* __restrict__ dst, long long shard4, float scale,
                                                       int rank, int world, int channel, uint32_t epoch,
                                                       uint32_t* gate, int* status) {
  vb_jitter(4u);
  if (!grid_enter(pads, rank, world, channel, epoch, gate, status)) return;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < shard4; i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int q = 0; q < world; ++q) {
      const int p = (rank + q) % world;
      const float4 v = *(reinterpret_cast<const float4*>(fulls.p[p]) + full_off4 + (long long)rank * shard4 + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float4 d = dst[i];
    d.x += scale * acc.x; d.y += scale * acc.y; d.z += scale * acc.z; d.w += scale * acc.w;
    dst[i] = d;
  }
}

// GEMM -> reduce-scatter, second half. slots = this rank's receive buffer [world, n] (bf16 or fp32; slot s was
// written by rank s's GEMM epilogue over NVLink). After the handshake (every rank's GEMM has finished, so all slots
// are complete) out[i] = sum_s slots[s][i] (+ residual[i]), fp32 accumulation in rank order. Local reads only.
template <typename T>
__global__ void peer_sum_slots_kernel(const T* __restrict__ slots, PeerPtrs pads, T* __restrict__ out,
                                      const T* __restrict__ residual, long long n, int rank, int world, int channel,
                                      uint32_t epoch, uint32_t* gate, int* status) {
  vb_jitter(5u);
  if (!grid_enter(pads, rank, world, channel, epoch, gate, status)) return;
  constexpr int V = 16 / sizeof(T);
  const long long n_vec = n / V;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    if (residual != nullptr) {
      const uint4 rv = reinterpret_cast<const uint4*>(residual)[i];
      const T* rp = reinterpret_cast<const T*>(&rv);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = to_float(rp[j]);
    }
    for (int s = 0; s < world; ++s) {
      const uint4 v = reinterpret_cast<const uint4*>(slots + (long long)s * n)[i];
      const T* vp = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += to_float(vp[j]);
    }
    uint4 o;
    T* op = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < V; ++j) op[j] = from_float<T>(acc[j]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

// Same reduction through the NVSwitch: one multimem.ld_reduce returns the sum over all ranks' copies.
__global__ void nvls_reduce_scatter_add_kernel(const float* mc_base, PeerPtrs pads, long long full_off4,
                                               float4* __restrict__ dst, long long shard4, float scale, int rank,
                                               int world, int channel, uint32_t epoch, uint32_t* gate, int* status) {
  vb_jitter(6u);
  if (!grid_enter(pads, rank, world, channel, epoch, gate, status)) return;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float4* src = reinterpret_cast<const float4*>(mc_base) + full_off4 + (long long)rank * shard4;
  constexpr int U = 4;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < shard4; i0 += stride * U) {
    float4 acc[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < shard4)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(acc[u].x), "=f"(acc[u].y), "=f"(acc[u].z), "=f"(acc[u].w)
                     : "l"(src + i)
                     : "memory");
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < shard4) {
        float4 d = dst[i];
        d.x += scale * acc[u].x; d.y += scale * acc[u].y; d.z += scale * acc[u].z; d.w += scale * acc[u].w;
        dst[i] = d;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Tensor-parallel row-parallel epilogue in one launch: all-reduce + residual add + RMSNorm.
//
// Every rank's GEMM has written its partial product [rows, H] (bf16) at the same offset of its symmetric buffer. After
// the cross-rank handshake each rank pulls all partials over NVLink (all ranks' loads in flight), adds them in rank
// order in fp32 (+ the residual stream), so that every rank gets bit-identical sums, writes the new residual stream and,
// when w != nullptr, the RMS-normalised row for the next column-parallel GEMM.
//
// The epoch of this channel lives on the device (*epoch_ctr) and is advanced by the last block to leave, so the same
// launch can be replayed from a CUDA graph; the channel must not be shared with launchers that pass epochs from the host.
// The partial buffer may be rewritten once a LATER handshake of this channel has passed on this rank (callers alternate
// two buffers).
template <int W>
__global__ void tp_allreduce_rmsnorm_kernel(PeerPtrs partials, PeerPtrs pads, long long off16,
                                            const __nv_bfloat16* __restrict__ residual_in,
                                            const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ normed,
                                            __nv_bfloat16* __restrict__ residual_out, int rows, int H, float eps, int rank,
                                            int world, int channel, uint32_t* epoch_ctr, uint32_t* done_ctr,
                                            uint32_t* gate, int* status) {
  vb_jitter(7u);
  extern __shared__ uint4 row_s[];  // H / 8 vectors: the summed row as bf16
  __shared__ float red_s[32];
  __shared__ uint32_t epoch_s;
  if (threadIdx.x == 0) epoch_s = *reinterpret_cast<volatile uint32_t*>(epoch_ctr) + 1u;
  __syncthreads();
  const uint32_t epoch = epoch_s;
  const bool ok = grid_enter(pads, rank, world, channel, epoch, gate, status);
  if (ok) {
    const int nvec = H >> 3;
    const uint4* src[W];
#pragma unroll
    for (int q = 0; q < W; ++q) src[q] = reinterpret_cast<const uint4*>(partials.p[q]) + off16;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
      const long long base = (long long)row * nvec;
      float ss = 0.f;
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        uint4 pv[W];
#pragma unroll
        for (int q = 0; q < W; ++q) pv[q] = src[q][base + v];
        float acc[8];
        if (residual_in != nullptr) {
          const uint4 rv = reinterpret_cast<const uint4*>(residual_in)[base + v];
          const __nv_bfloat16* rp = reinterpret_cast<const __nv_bfloat16*>(&rv);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = __bfloat162float(rp[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        }
#pragma unroll
        for (int q = 0; q < W; ++q) {
          const __nv_bfloat16* pp = reinterpret_cast<const __nv_bfloat16*>(&pv[q]);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(pp[j]);
        }
        uint4 o;
        __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          op[j] = __float2bfloat16(acc[j]);
          const float r = __bfloat162float(op[j]);  // the norm sees exactly what later layers will read
          ss += r * r;
        }
        row_s[v] = o;
        reinterpret_cast<uint4*>(residual_out)[base + v] = o;
      }
      if (w != nullptr) {
        ss = warp_reduce_sum(ss);
        if ((threadIdx.x & 31) == 0) red_s[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red_s[i];
        const float rstd = rsqrtf(tot / H + eps);
        for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
          const uint4 hv = row_s[v];
          const uint4 wv = reinterpret_cast<const uint4*>(w)[v];
          const __nv_bfloat16* hp = reinterpret_cast<const __nv_bfloat16*>(&hv);
          const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(&wv);
          uint4 o;
          __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
          for (int j = 0; j < 8; ++j) op[j] = __float2bfloat16(__bfloat162float(hp[j]) * rstd * __bfloat162float(wp[j]));
          reinterpret_cast<uint4*>(normed)[base + v] = o;
        }
        __syncthreads();  // red_s and row_s are reused by the next row
      }
    }
  }
  // leave: the last block advances the epoch for the next launch (also after a failed handshake, so that the counters
  // of a later attempt start from a consistent state)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      *done_ctr = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(epoch_ctr) = epoch;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// All-to-all of row chunks over peer memory (the Ulysses exchanges around attention: gather the sequence and scatter
// the heads, and back). Every rank has staged its tensor in symmetric memory; after the handshake each rank PULLS, from
// every rank r, `rows` chunks of `chunk16` 16-byte units: chunk t of rank r starts at src_base16[r] + t * src_stride16
// in r's buffer and lands at dst_base16[r] + t * dst_stride16 locally, i.e. directly in the layout the attention (or the
// projection after it) wants: no intermediate buffers, no concatenation pass.
struct A2AParams {
  long long src_base16[MAX_RANKS];
  long long dst_base16[MAX_RANKS];
  long long src_stride16, dst_stride16;
  int rows, chunk16;
};

__global__ void peer_a2a_chunks_kernel(PeerPtrs srcs, PeerPtrs pads, long long src_off16, uint4* __restrict__ dst,
                                       A2AParams q, int rank, int world, int channel, uint32_t epoch, uint32_t* gate,
                                       int* status) {
  vb_jitter(8u);
  if (!grid_enter(pads, rank, world, channel, epoch, gate, status)) return;
  const long long per_rank = (long long)q.rows * q.chunk16;
  const long long total = per_rank * world;
  const long long stride = (long long)gridDim.x * blockDim.x;
  constexpr int U = 4;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < total; i0 += stride * U) {
    uint4 v[U];
    long long d[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      d[u] = -1;
      if (i < total) {
        const int rr = (int)(i / per_rank);
        const int r = (rr + rank) % world;  // start every rank on a different peer
        const long long w = i - (long long)rr * per_rank;
        const long long t = w / q.chunk16, c = w - t * q.chunk16;
        v[u] = (reinterpret_cast<const uint4*>(srcs.p[r]) + src_off16)[q.src_base16[r] + t * q.src_stride16 + c];
        d[u] = q.dst_base16[r] + t * q.dst_stride16 + c;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (d[u] >= 0) dst[d[u]] = v[u];
  }
}

struct Segment {
  long long src_off;  // bytes from the base of the source rank's symmetric buffer (16-byte aligned)
  long long dst_off;  // bytes from dst_base (16-byte aligned)
  long long nbytes;   // multiple of 16
  int src_rank;
  int pad;
};

// One block walks whole segments (grid-stride over the table); large segments are split by the planner.
__global__ void peer_segment_copy_kernel(PeerPtrs srcs, PeerPtrs pads, const Segment* __restrict__ segs, int nseg,
                                         uint8_t* __restrict__ dst_base, int rank, int world, int channel,
                                         uint32_t epoch, uint32_t* gate, int* status) {
  vb_jitter(9u);
  if (!grid_enter(pads, rank, world, channel, epoch, gate, status)) return;
  for (int s = blockIdx.x; s < nseg; s += gridDim.x) {
    const Segment sg = segs[s];
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(srcs.p[sg.src_rank]) + sg.src_off);
    uint4* dst = reinterpret_cast<uint4*>(dst_base + sg.dst_off);
    const long long n16 = sg.nbytes >> 4;
    constexpr int U = 4;
    for (long long i0 = threadIdx.x; i0 < n16; i0 += (long long)blockDim.x * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + (long long)u * blockDim.x;
        if (i < n16) v[u] = src[i];
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + (long long)u * blockDim.x;
        if (i < n16) dst[i] = v[u];
      }
    }
  }
}

static PeerPtrs make_ptrs(const void* const* arr, int world) {
  PeerPtrs pp{};
  for (int i = 0; i < world && i < MAX_RANKS; ++i) pp.p[i] = const_cast<void*>(arr[i]);
  return pp;
}

}  // namespace vb

using namespace vb;

extern "C" int vb_peer_max_ranks() { return MAX_RANKS; }

extern "C" int vb_peer_barrier(const void* const* pads, int rank, int world, int channel, unsigned epoch, int* status,
                               cudaStream_t stream) {
  if (world > MAX_RANKS) return -3;
  peer_barrier_kernel<<<1, 32, 0, stream>>>(make_ptrs(pads, world), rank, world, channel, epoch, status);
  vb_count_launch();
  return (int)cudaGetLastError();
}

// All byte counts / offsets must be multiples of 16. `gate` is a device uint32 owned by the caller (per channel).
extern "C" int vb_peer_all_gather(const void* const* srcs, const void* const* pads, long long src_off_bytes, void* out,
                                  long long shard_bytes, int rank, int world, int channel, unsigned epoch,
                                  unsigned* gate, int* status, cudaStream_t stream) {
  if (world > MAX_RANKS || (src_off_bytes & 15) || (shard_bytes & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return -3;
  const long long total16 = (shard_bytes >> 4) * world;
  long long blocks = (total16 + 255) / 256;
  const int cap = vb_num_sms();  // all blocks must be co-resident with block 0: at most one wave
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  peer_all_gather_kernel<<<(int)blocks, 256, 0, stream>>>(make_ptrs(srcs, world), make_ptrs(pads, world),
                                                          src_off_bytes >> 4, reinterpret_cast<uint4*>(out),
                                                          shard_bytes >> 4, rank, world, channel, epoch, gate, status);
  vb_count_launch();
  return (int)cudaGetLastError();
}

// The same all-gather with the payload moved by the copy engines: a one-block kernel does the cross-rank
// handshake (every rank's shard is final), then one asynchronous copy per peer pulls the shards over NVLink
// without occupying SMs, so a gather issued on a side stream does not slow the GEMMs it overlaps.
extern "C" int vb_peer_all_gather_ce(const void* const* srcs, const void* const* pads, long long src_off_bytes,
                                     void* out, long long shard_bytes, int rank, int world, int channel,
                                     unsigned epoch, int* status, cudaStream_t stream) {
  if (world > MAX_RANKS) return -3;
  peer_barrier_kernel<<<1, 32, 0, stream>>>(make_ptrs(pads, world), rank, world, channel, epoch, status);
  vb_count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  for (int q = 0; q < world; ++q) {
    const int p = (rank + 1 + q) % world;  // own shard last
    e = cudaMemcpyAsync(reinterpret_cast<uint8_t*>(out) + (long long)p * shard_bytes,
                        reinterpret_cast<const uint8_t*>(srcs[p]) + src_off_bytes, (size_t)shard_bytes,
                        cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

extern "C" int vb_peer_reduce_scatter_add(const void* const* fulls, const void* const* pads, const void* mc_base,
                                          long long full_off_bytes, float* dst, long long shard_floats, float scale,
                                          int rank, int world, int channel, unsigned epoch, unsigned* gate, int* status,
                                          cudaStream_t stream) {
  if (world > MAX_RANKS || (full_off_bytes & 15) || (shard_floats & 3) || (reinterpret_cast<uintptr_t>(dst) & 15)) return -3;
  const long long shard4 = shard_floats >> 2;
  long long blocks = (shard4 + 1023) / 1024;
  const int cap = 2 * vb_num_sms();  // all blocks must be co-resident with block 0: two small blocks per SM always fit
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (mc_base != nullptr) {
    nvls_reduce_scatter_add_kernel<<<(int)blocks, 256, 0, stream>>>(
        reinterpret_cast<const float*>(mc_base), make_ptrs(pads, world), full_off_bytes >> 4,
        reinterpret_cast<float4*>(dst), shard4, scale, rank, world, channel, epoch, gate, status);
  } else {
#define VB_RS_ARGS make_ptrs(fulls, world), make_ptrs(pads, world), full_off_bytes >> 4, reinterpret_cast<float4*>(dst), \
                   shard4, scale, rank, world, channel, epoch, gate, status
    if (world == 2) peer_reduce_scatter_add_kernel<2, 4><<<(int)blocks, 256, 0, stream>>>(VB_RS_ARGS);
    else if (world == 4) peer_reduce_scatter_add_kernel<4, 2><<<(int)blocks, 256, 0, stream>>>(VB_RS_ARGS);
    else if (world == 8) peer_reduce_scatter_add_kernel<8, 2><<<(int)blocks, 256, 0, stream>>>(VB_RS_ARGS);
    else peer_reduce_scatter_add_generic_kernel<<<(int)blocks, 256, 0, stream>>>(VB_RS_ARGS);
#undef VB_RS_ARGS
  }
  vb_count_launch();
  return (int)cudaGetLastError();
}

extern "C" int vb_peer_sum_slots(const void* slots, const void* const* pads, void* out, const void* residual,
                                 long long n, int fp32, int rank, int world, int channel, unsigned epoch,
                                 unsigned* gate, int* status, cudaStream_t stream) {
  if (world > MAX_RANKS || n <= 0 || (n % (fp32 ? 4 : 8)) != 0) return -3;
  const long long n_vec = n / (fp32 ? 4 : 8);
  long long blocks = (n_vec + 255) / 256;
  const long long cap = 4LL * vb_num_sms();
  if (blocks > cap) blocks = cap;
  if (fp32) {
    peer_sum_slots_kernel<float><<<(int)blocks, 256, 0, stream>>>(
        reinterpret_cast<const float*>(slots), make_ptrs(pads, world), reinterpret_cast<float*>(out),
        reinterpret_cast<const float*>(residual), n, rank, world, channel, epoch, gate, status);
  } else {
    peer_sum_slots_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(slots), make_ptrs(pads, world), reinterpret_cast<__nv_bfloat16*>(out),
        reinterpret_cast<const __nv_bfloat16*>(residual), n, rank, world, channel, epoch, gate, status);
  }
  vb_count_launch();
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------------------
// Expert-parallel MoE: dispatch (push) and combine (pull) over peer memory.
//
// Rank r owns experts [r * E_local, (r + 1) * E_local). The host side has all-gathered the per-rank expert histograms,
// so every rank knows where its rows of expert e start in the owner's receive buffer (base[e]); the buffer is laid out
// exactly as the grouped GEMM wants it (rows sorted by expert, every expert padded to 128 rows), so the owner runs its
// experts on the received rows without sorting them.
//   dispatch: one warp per (token, slot) pair claims the next row of its expert's sub-range (local atomic) and stores
//             the token's hidden vector there with 512-byte warp stores over NVLink; `where` remembers the row.
//   combine:  after a bounded cross-rank handshake (all owners have finished their experts), one warp per token loads
//             its k expert outputs from the owners' buffers (all k loads in flight) and writes the weighted sum.
__global__ void moe_dispatch_kernel(const uint4* __restrict__ x, const int* __restrict__ top_i, int pairs, int k,
                                    int h16, int e_local, const int* __restrict__ base, int* __restrict__ cursor,
                                    PeerPtrs recv, int* __restrict__ where, long long cap_rows, int* status) {
  vb_jitter(10u);
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int pair = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; pair < pairs; pair += warps) {
    const int e = top_i[pair];
    int pos = 0;
    if (lane == 0) pos = base[e] + atomicAdd(cursor + e, 1);
    pos = __shfl_sync(0xffffffffu, pos, 0);
    if (pos < 0 || pos >= cap_rows) {  // the receive buffer is too small for this routing: refuse, do not write
      if (lane == 0) {
        report_error(status, ERR_BAD_ARG, pair);
        where[pair] = -1;
      }
      continue;
    }
    const uint4* src = x + (long long)(pair / k) * h16;
    uint4* dst = reinterpret_cast<uint4*>(recv.p[e / e_local]) + (long long)pos * h16;
    for (int i = lane; i < h16; i += 32) dst[i] = src[i];
    if (lane == 0) where[pair] = pos;
  }
}

// Histogram of this rank's routing (one block): hist[e] = number of (token, slot) pairs routed to expert e.
__global__ void moe_hist_kernel(const int* __restrict__ top_i, int pairs, int num_experts, int* __restrict__ hist) {
  vb_jitter(11u);
  extern __shared__ int h_s[];
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) h_s[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = top_i[i];
    if (e >= 0 && e < num_experts) atomicAdd(h_s + e, 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) hist[e] = h_s[e];
}

// From the all-gathered histograms hist_all [world, hist_stride] (one block): base[e] = first row, in the owner's
// receive buffer, of this rank's rows of expert e; expert_off [e_local + 1] and blk_expert [blocks] describe the rows
// this rank receives (every expert padded to 128 rows; blocks past the end are -1); cursor [E] is zeroed.
__global__ void moe_layout_kernel(const int* __restrict__ hist_all, int hist_stride, int num_experts, int e_local,
                                  int rank, int world, int* __restrict__ base, int* __restrict__ expert_off,
                                  int* __restrict__ blk_expert, int blocks, int* __restrict__ cursor) {
  vb_jitter(12u);
  extern __shared__ int l_s[];
  int* padded = l_s;                 // [E]
  int* off = l_s + num_experts;      // [E] owner-local first row of every expert
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    int tot = 0;
    for (int s2 = 0; s2 < world; ++s2) tot += hist_all[s2 * hist_stride + e];
    padded[e] = (tot + 127) / 128 * 128;
    cursor[e] = 0;
  }
  __syncthreads();
  for (int o = threadIdx.x; o < world; o += blockDim.x) {  // one thread per owner: serial scan of its experts
    int run = 0;
    for (int j = 0; j < e_local; ++j) {
      off[o * e_local + j] = run;
      run += padded[o * e_local + j];
    }
    if (o == rank) expert_off[e_local] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    int before = 0;
    for (int s2 = 0; s2 < rank; ++s2) before += hist_all[s2 * hist_stride + e];
    base[e] = off[e] + before;
    if (e / e_local == rank) expert_off[e - rank * e_local] = off[e];
  }
  const int* my_off = off + rank * e_local;
  const int* my_pad = padded + rank * e_local;
  for (int b = threadIdx.x; b < blocks; b += blockDim.x) {
    const int r0 = b * 128;
    int found = -1;
    for (int j = 0; j < e_local; ++j)
      if (r0 >= my_off[j] && r0 < my_off[j] + my_pad[j]) found = j;
    blk_expert[b] = found;
  }
}

extern "C" int vb_moe_hist(const int* top_i, int pairs, int num_experts, int* hist, cudaStream_t stream) {
  if (num_experts < 1 || num_experts > 8192) return -3;
  moe_hist_kernel<<<1, 1024, num_experts * sizeof(int), stream>>>(top_i, pairs, num_experts, hist);
  vb_count_launch();
  return (int)cudaGetLastError();
}

extern "C" int vb_moe_layout(const int* hist_all, int hist_stride, int num_experts, int e_local, int rank, int world,
                             int* base, int* expert_off, int* blk_expert, int blocks, int* cursor,
                             cudaStream_t stream) {
  if (num_experts < 1 || num_experts > 4096 || e_local * world != num_experts) return -3;
  moe_layout_kernel<<<1, 256, 2 * num_experts * sizeof(int), stream>>>(hist_all, hist_stride, num_experts, e_local, rank,
                                                                      world, base, expert_off, blk_expert, blocks, cursor);
  vb_count_launch();
  return (int)cudaGetLastError();
}

template <int KMAX>
__global__ void moe_combine_kernel(PeerPtrs y, PeerPtrs pads, const int* __restrict__ top_i,
                                   const float* __restrict__ top_w, const int* __restrict__ where, int tokens, int k,
                                   int h16, int e_local, uint4* __restrict__ out, int rank, int world, int channel,
                                   uint32_t epoch, uint32_t* gate, int* status) {
  vb_jitter(13u);
  if (!grid_enter(pads, rank, world, channel, epoch, gate, status)) return;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < tokens; t += warps) {
    const uint4* rowp[KMAX];
    float w[KMAX];
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      rowp[j] = nullptr;
      w[j] = 0.f;
      if (j < k) {
        const int row = where[t * k + j];
        if (row >= 0) {
          rowp[j] = reinterpret_cast<const uint4*>(y.p[top_i[t * k + j] / e_local]) + (long long)row * h16;
          w[j] = top_w[t * k + j];
        }
      }
    }
    for (int i = lane; i < h16; i += 32) {
      uint4 v[KMAX];
#pragma unroll
      for (int j = 0; j < KMAX; ++j) v[j] = rowp[j] != nullptr ? rowp[j][i] : make_uint4(0u, 0u, 0u, 0u);
      float acc[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.f;
#pragma unroll
      for (int j = 0; j < KMAX; ++j) {
        const __nv_bfloat16* hp = reinterpret_cast<const __nv_bfloat16*>(&v[j]);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] += w[j] * __bfloat162float(hp[q]);
      }
      uint4 o;
      __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
      for (int q = 0; q < 8; ++q) op[q] = __float2bfloat16(acc[q]);
      out[(long long)t * h16 + i] = o;
    }
  }
}

extern "C" int vb_moe_dispatch(const void* x, const int* top_i, int tokens, int k, int hidden, int e_local,
                               const int* base, int* cursor, const void* const* recv, int world, int* where,
                               long long cap_rows, int* status, cudaStream_t stream) {
  if (world > MAX_RANKS || (hidden & 7) || k < 1 || e_local < 1) return -3;
  const int pairs = tokens * k;
  if (pairs <= 0) return 0;
  int blocks = (pairs + 7) / 8;  // 8 warps per block
  const int cap = 8 * vb_num_sms();
  if (blocks > cap) blocks = cap;
  moe_dispatch_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint4*>(x), top_i, pairs, k, hidden / 8, e_local,
                                                  base, cursor, make_ptrs(recv, world), where, cap_rows, status);
  vb_count_launch();
  return (int)cudaGetLastError();
}

extern "C" int vb_moe_combine(const void* const* y, const void* const* pads, const int* top_i, const float* top_w,
                              const int* where, int tokens, int k, int hidden, int e_local, void* out, int rank,
                              int world, int channel, unsigned epoch, unsigned* gate, int* status,
                              cudaStream_t stream) {
  if (world > MAX_RANKS || (hidden & 7) || k < 1 || k > 8 || e_local < 1) return -3;
  int blocks = (tokens + 7) / 8;
  const int cap = 8 * vb_num_sms();
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;  // the handshake must run even when this rank has no tokens
#define VB_COMBINE(KM)                                                                                              \
  moe_combine_kernel<KM><<<blocks, 256, 0, stream>>>(make_ptrs(y, world), make_ptrs(pads, world), top_i, top_w, where, \
                                                     tokens, k, hidden / 8, e_local, reinterpret_cast<uint4*>(out), rank, \
                                                     world, channel, epoch, gate, status)
  if (k <= 2) VB_COMBINE(2);
  else if (k <= 4) VB_COMBINE(4);
  else VB_COMBINE(8);
#undef VB_COMBINE
  vb_count_launch();
  return (int)cudaGetLastError();
}

// partials[r] = base of rank r's symmetric buffer, the partial product sits at byte offset `off_bytes` in each of them.
// ctrs: three device words owned by the caller for this channel (epoch, done counter, gate), zero before first use.
extern "C" int vb_tp_allreduce_rmsnorm(const void* const* partials, const void* const* pads, long long off_bytes,
                                       const void* residual_in, const void* w, void* normed, void* residual_out, int rows,
                                       int H, float eps, int rank, int world, int channel, unsigned* ctrs, int* status,
                                       cudaStream_t stream) {
  if (world > MAX_RANKS || (H & 7) || (off_bytes & 15) || rows <= 0 || residual_out == nullptr) return -3;
  if (w != nullptr && normed == nullptr) return -3;
  int blocks = rows;
  const int cap = 4 * vb_num_sms();  // every block must be resident while block 0 runs the handshake
  if (blocks > cap) blocks = cap;
  const int threads = H >= 4096 ? 512 : 256;
  const size_t smem = (size_t)H * 2;
  if (smem > 48 * 1024) return -3;
#define VB_TPAR(WV)                                                                                                  \
  tp_allreduce_rmsnorm_kernel<WV><<<blocks, threads, smem, stream>>>(                                                \
      make_ptrs(partials, world), make_ptrs(pads, world), off_bytes >> 4,                                            \
      reinterpret_cast<const __nv_bfloat16*>(residual_in), reinterpret_cast<const __nv_bfloat16*>(w),                \
      reinterpret_cast<__nv_bfloat16*>(normed), reinterpret_cast<__nv_bfloat16*>(residual_out), rows, H, eps, rank,  \
      world, channel, ctrs, ctrs + 1, ctrs + 2, status)
  if (world == 2) VB_TPAR(2);
  else if (world == 4) VB_TPAR(4);
  else if (world == 8) VB_TPAR(8);
  else return -3;
#undef VB_TPAR
  vb_count_launch();
  return (int)cudaGetLastError();
}

// src_base / dst_base: `world` offsets each, strides and chunk in units of 16 bytes (see peer_a2a_chunks_kernel).
extern "C" int vb_peer_a2a_chunks(const void* const* srcs, const void* const* pads, long long src_off_bytes, void* dst,
                                  const long long* src_base16, const long long* dst_base16, long long src_stride16,
                                  long long dst_stride16, int rows, int chunk16, int rank, int world, int channel,
                                  unsigned epoch, unsigned* gate, int* status, cudaStream_t stream) {
  if (world > MAX_RANKS || (src_off_bytes & 15) || rows < 0 || chunk16 <= 0 || (reinterpret_cast<uintptr_t>(dst) & 15)) return -3;
  A2AParams q{};
  for (int r = 0; r < world; ++r) {
    q.src_base16[r] = src_base16[r];
    q.dst_base16[r] = dst_base16[r];
  }
  q.src_stride16 = src_stride16;
  q.dst_stride16 = dst_stride16;
  q.rows = rows;
  q.chunk16 = chunk16;
  const long long total = (long long)rows * chunk16 * world;
  long long blocks = (total + 1023) / 1024;
  const int cap = 2 * vb_num_sms();  // every block must be resident while block 0 runs the handshake
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  peer_a2a_chunks_kernel<<<(int)blocks, 256, 0, stream>>>(make_ptrs(srcs, world), make_ptrs(pads, world), src_off_bytes >> 4,
                                                          reinterpret_cast<uint4*>(dst), q, rank, world, channel, epoch,
                                                          gate, status);
  vb_count_launch();
  return (int)cudaGetLastError();
}

// segs: device array of {int64 src_off, int64 dst_off, int64 nbytes, int32 src_rank, int32 pad} (32 bytes each).
extern "C" int vb_peer_segment_copy(const void* const* srcs, const void* const* pads, const void* segs, int nseg,
                                    void* dst_base, int rank, int world, int channel, unsigned epoch, unsigned* gate,
                                    int* status, cudaStream_t stream) {
  if (world > MAX_RANKS) return -3;
  if (nseg <= 0) return 0;
  int blocks = nseg < vb_num_sms() ? nseg : vb_num_sms();
  peer_segment_copy_kernel<<<blocks, 512, 0, stream>>>(make_ptrs(srcs, world), make_ptrs(pads, world),
                                                       reinterpret_cast<const Segment*>(segs), nseg,
                                                       reinterpret_cast<uint8_t*>(dst_base), rank, world, channel, epoch,
                                                       gate, status);
  vb_count_launch();
  return (int)cudaGetLastError();
}
