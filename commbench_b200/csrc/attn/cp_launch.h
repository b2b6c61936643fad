// Host-side interface between the planners (ring.cu, ulysses.cu) and the kernel (fa_cp.cu).
#pragma once
#include <cuda_runtime.h>

#include "fa_cp_types.h"

namespace cb {

// Launches fa_cp_kernel with `grid` CTAs (communication tickets + attention items).
int cp_launch(const FaCpParams& p, int grid, cudaStream_t st);

// Attention items of a parameter block: tile pairs of all query segments x heads x batch.
int cp_num_items(const FaCpParams& p);

}  // namespace cb

// [rows, heads, 128] bf16 tensor map with 64 x 1 x 128 boxes (fa_fwd.cu).
int cb_attn_make_tmap_bshd(CUtensorMap* out, const void* base, int rows, int heads);
