// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled), with the
// alignment rules checked up front so that a bad argument becomes an error
// string instead of a device fault.
#pragma once
#include <cuda.h>

#include <string>

namespace cb {

enum TmapDtype { TMAP_BF16 = 0, TMAP_U8 = 1, TMAP_F32 = 2 };

// 2-D row-major tensor [outer][inner]; box = [box_outer][box_inner]; 128-byte
// swizzle when `swizzle128` (box_inner * elem must then be exactly 128 bytes).
// Returns 0 or -1 (reason through set_last_error).
int make_tmap_2d(CUtensorMap* out, const void* base, TmapDtype dt, unsigned long long inner,
                 unsigned long long outer, unsigned long long row_stride_bytes,
                 unsigned box_inner, unsigned box_outer, bool swizzle128);

}  // namespace cb
