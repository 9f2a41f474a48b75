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
