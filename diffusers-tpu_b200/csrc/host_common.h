// Host-side helpers shared by the C-ABI translation units: status mapping, the
// driver entry point for tensor-map encoding, and the [B,H,S,D] bf16 tensor map.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/dtb200_attn.h"

namespace dtb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

// Resolved once; the driver symbol is reached through the runtime so the library
// does not link against libcuda directly.
EncodeTiledFn get_encode_tiled();

// Tensor map over a bf16 [B, H, S, 128] tensor with element strides (sb, sh, ss, 1):
// boxes of 64 (head_dim) x `box_rows` (sequence) elements, 128-byte swizzle, zero fill
// outside the tensor.  Returns a dtb_status.
int make_tmap_bhsd(CUtensorMap* out, const void* base, int64_t B, int64_t H, int64_t S, int64_t sb,
                   int64_t sh, int64_t ss, int box_rows);

// Same for an 8-bit (E4M3) [B, H, S, 128] tensor: boxes of 128 bytes x `box_rows`.
int make_tmap_bhsd_u8(CUtensorMap* out, const void* base, int64_t B, int64_t H, int64_t S, int64_t sb, int64_t sh,
                      int64_t ss, int box_rows);

// Tensor map over a row-major bf16 matrix [rows, cols] (row stride in elements): boxes of `box_cols` (<= 64)
// columns x `box_rows` rows, 128-byte swizzle, zero fill outside the matrix.
int make_tmap_rows_bf16(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t row_stride,
                        int box_rows, int box_cols);

// Records the CUDA error behind a DTB_ERR_LAUNCH so that dtb_last_error_detail() can name it.
// Returns true when `e` is cudaSuccess.
bool cuda_ok(cudaError_t e, const char* what);
// Checks (and clears) the launch error of the kernel just enqueued.
bool launch_ok(const char* what);
const char* last_detail();
// Sets the text dtb_last_error_detail() returns for the calling thread.
void set_detail(const char* text);

// True when the current device is compute capability 10.x.
bool device_is_sm100();

}  // namespace dtb
