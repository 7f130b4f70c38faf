#include "host_common.h"

#include <cstdio>
#include <mutex>

namespace dtb {

namespace {
thread_local char g_detail[256] = "";
}

bool cuda_ok(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return true;
  snprintf(g_detail, sizeof(g_detail), "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
  (void)cudaGetLastError();
  return false;
}

bool launch_ok(const char* what) { return cuda_ok(cudaGetLastError(), what); }

const char* last_detail() { return g_detail; }

void set_detail(const char* text) { snprintf(g_detail, sizeof(g_detail), "%s", text); }

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
    (void)cudaGetLastError();
  });
  return fn;
}

namespace {
int encode_bhsd(CUtensorMap* out, const void* base, int64_t B, int64_t H, int64_t S, int64_t sb, int64_t sh, int64_t ss,
                int box_rows, int64_t esz);
}

int make_tmap_bhsd(CUtensorMap* out, const void* base, int64_t B, int64_t H, int64_t S, int64_t sb,
                   int64_t sh, int64_t ss, int box_rows) {
  return encode_bhsd(out, base, B, H, S, sb, sh, ss, box_rows, 2);
}

int make_tmap_bhsd_u8(CUtensorMap* out, const void* base, int64_t B, int64_t H, int64_t S, int64_t sb, int64_t sh,
                      int64_t ss, int box_rows) {
  return encode_bhsd(out, base, B, H, S, sb, sh, ss, box_rows, 1);
}

namespace {
int encode_bhsd(CUtensorMap* out, const void* base, int64_t B, int64_t H, int64_t S, int64_t sb, int64_t sh, int64_t ss,
                int box_rows, int64_t esz) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) {
    snprintf(g_detail, sizeof(g_detail), "cuTensorMapEncodeTiled entry point not found");
    return DTB_ERR_LAUNCH;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return DTB_ERR_ALIGN;
  if (((ss * esz) & 15) || (H > 1 && ((sh * esz) & 15)) || (B > 1 && ((sb * esz) & 15))) return DTB_ERR_ALIGN;
  // An axis of extent > 1 needs a positive stride: a broadcast (stride 0) or reversed view cannot be described
  // to TMA, and substituting a stride would read the wrong memory.
  if (ss <= 0 || (H > 1 && sh <= 0) || (B > 1 && sb <= 0)) return DTB_ERR_SHAPE;
  cuuint64_t gdim[4] = {128, static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(H),
                        static_cast<cuuint64_t>(B)};
  // A size-1 axis may come with any stride (torch reports arbitrary values there);
  // give it a harmless legal one.
  cuuint64_t gstr[3] = {static_cast<cuuint64_t>(ss * esz),
                        static_cast<cuuint64_t>((H > 1 ? sh : S * ss) * esz),
                        static_cast<cuuint64_t>((B > 1 ? sb : H * S * ss) * esz)};
  if (H == 1 && (gstr[1] == 0 || (gstr[1] & 15))) gstr[1] = 256;
  if (B == 1 && (gstr[2] == 0 || (gstr[2] & 15))) gstr[2] = 256;
  cuuint32_t box[4] = {static_cast<cuuint32_t>(128 / esz), static_cast<cuuint32_t>(box_rows), 1, 1};   // 128-byte rows
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 4,
                   const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_detail, sizeof(g_detail), "cuTensorMapEncodeTiled failed with CUresult %d (S=%lld H=%lld B=%lld)",
             static_cast<int>(r), static_cast<long long>(S), static_cast<long long>(H), static_cast<long long>(B));
    return DTB_ERR_LAUNCH;
  }
  return DTB_OK;
}
}  // namespace

int make_tmap_rows_bf16(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t row_stride,
                        int box_rows, int box_cols) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) {
    snprintf(g_detail, sizeof(g_detail), "cuTensorMapEncodeTiled entry point not found");
    return DTB_ERR_LAUNCH;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || ((row_stride * 2) & 15)) return DTB_ERR_ALIGN;
  if (rows <= 0 || cols <= 0 || row_stride < cols || box_cols > 64 || box_rows > 256) return DTB_ERR_SHAPE;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstr[1] = {static_cast<cuuint64_t>(row_stride * 2)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_detail, sizeof(g_detail), "cuTensorMapEncodeTiled (2-D) failed with CUresult %d (rows=%lld cols=%lld)",
             static_cast<int>(r), static_cast<long long>(rows), static_cast<long long>(cols));
    return DTB_ERR_LAUNCH;
  }
  return DTB_OK;
}

bool device_is_sm100() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return false;
  return major == 10;
}

}  // namespace dtb

extern "C" int dtb_version(void) { return 100; }

extern "C" const char* dtb_last_error_detail(void) { return dtb::last_detail(); }

extern "C" const char* dtb_status_string(int status) {
  switch (status) {
    case DTB_OK: return "ok";
    case DTB_ERR_NULL: return "a required pointer is NULL";
    case DTB_ERR_DTYPE: return "unsupported element type";
    case DTB_ERR_SHAPE: return "unsupported shape";
    case DTB_ERR_ALIGN: return "pointer or stride is not 16-byte aligned";
    case DTB_ERR_ARCH: return "device is not sm_100";
    case DTB_ERR_WORKSPACE: return "workspace missing or too small";
    case DTB_ERR_LAUNCH: return "CUDA error while encoding tensor maps or launching";
    case DTB_ERR_TIMEOUT: return "a bounded device wait ran out";
    case DTB_ERR_UNSUPPORTED: return "unsupported option";
    default: return "unknown status";
  }
}
