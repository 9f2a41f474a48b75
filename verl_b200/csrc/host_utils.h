// Host helpers shared by the launchers of this library.
#pragma once
#include <cuda.h>
#include <stdint.h>

// 2-D tiled tensor map. `inner` is the contiguous dimension. The swizzle mode is
// chosen from the byte width of the box's inner extent (128/64/32 bytes).
// Returns 0 on success, a negative code otherwise.
int vb_make_tmap_2d(CUtensorMap* out, const void* ptr, int elem_bytes, uint64_t inner, uint64_t outer,
                    uint64_t outer_stride_bytes, uint32_t box_inner, uint32_t box_outer);
int vb_make_tmap_3d(CUtensorMap* out, const void* ptr, int elem_bytes, uint64_t d0, uint64_t d1, uint64_t d2,
                    uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2);
int vb_num_sms();

// 1 unless VERL_B200_PDL=0: kernels that call pdl_wait() are launched with the programmatic-serialization
// attribute, so that their prologue overlaps the tail of the kernel before them (inside CUDA graphs too).
int vb_pdl_enabled();

#ifdef __CUDACC__
#include <cuda_runtime.h>
// Launch `kern` (which must call vb::pdl_wait() before its first access to global memory) so that it may start
// before the previous kernel of the stream has finished. Cluster dimensions, when given, are attached as well.
template <typename... KArgs, typename... Args>
inline cudaError_t vb_launch_ex(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                unsigned cluster_x, bool pdl, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  unsigned n = 0;
  if (pdl && vb_pdl_enabled()) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = cluster_x;
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t vb_launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 unsigned cluster_x, Args&&... args) {
  return vb_launch_ex(kern, grid, block, smem, stream, cluster_x, true, static_cast<Args&&>(args)...);
}
#endif
