// Hardware self-tests for the encodings the attention kernels depend on.  Each
// test runs one CTA on one 128x128x128 tile and writes an f32 result the host
// compares with a plain matmul:
//   tmem_roundtrip : tcgen05.st -> tcgen05.ld lane/column mapping
//   qk             : TMA 128B-swizzled tiles + K-major smem descriptors (S = Q K^T)
//   pv             : bf16 A operand held in tensor memory + MN-major V descriptor (O = P V)
#include "host_common.h"
#include "ptx.cuh"

namespace dtb {
namespace {

constexpr int kTile = 128;
constexpr uint32_t kPanelBytes = kTile * 64 * 2;  // one 64-column panel of a 128-row tile

struct SelftestShared {
  uint64_t bar_load;
  uint64_t bar_mma;
  uint64_t bar_mma2;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint8_t* align_1024(uint8_t* p) {
  uint32_t a = smem_u32(p);
  return p + (((a + 1023u) & ~1023u) - a);
}

__global__ void __launch_bounds__(128) tmem_roundtrip_kernel(const float* __restrict__ in,
                                                             float* __restrict__ out, int* status) {
  __shared__ SelftestShared sh;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) sh.abort_flag = 0;
  if (warp == 0) {
    tmem_alloc(smem_u32(&sh.tmem_base), 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = sh.tmem_base;
  const int row = threadIdx.x;
  const uint32_t lane_addr = tbase + (static_cast<uint32_t>(warp * 32) << 16);
  uint32_t r[32];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(in[row * kTile + c * 32 + i]);
    tmem_st32(lane_addr + c * 32, r);
  }
  tmem_wait_st();
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    tmem_ld32(lane_addr + c * 32, r);
    tmem_wait_ld();
#pragma unroll
    for (int i = 0; i < 32; ++i) out[row * kTile + c * 32 + i] = __uint_as_float(r[i]);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 128);
  (void)status;
}

// mode 0: S = Q K^T with both operands from shared memory (K-major).
// mode 1: O = P V with P (bf16 pairs) in tensor memory and V MN-major in shared memory.
template <int kMode>
__global__ void __launch_bounds__(128) mma_tile_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                       const __grid_constant__ CUtensorMap tmap_b,
                                                       const __nv_bfloat16* __restrict__ a_global,
                                                       float* __restrict__ out, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ SelftestShared sh;
  uint8_t* smem = align_1024(smem_raw);
  uint8_t* smem_a = smem;                    // 32 KB: two 64-column panels
  uint8_t* smem_b = smem + 2 * kPanelBytes;  // 32 KB
  const int warp = threadIdx.x >> 5;
  AbortCtx ctx{&sh.abort_flag, status};

  if (threadIdx.x == 0) {
    sh.abort_flag = 0;
    mbar_init(smem_u32(&sh.bar_load), 1);
    mbar_init(smem_u32(&sh.bar_mma), 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&sh.tmem_base), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = sh.tmem_base;
  const uint32_t d_tmem = tbase;        // columns [0,128): f32 accumulator
  const uint32_t p_tmem = tbase + 128;  // columns [128,192): bf16 A operand (mode 1)
  const uint32_t lane_addr_off = static_cast<uint32_t>(warp * 32) << 16;

  if (kMode == 1) {
    // Every thread packs its row of P into 64 words and stores them to tensor memory.
    const __nv_bfloat16* prow = a_global + threadIdx.x * kTile;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t r[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        uint32_t lo = __bfloat16_as_ushort(prow[c * 64 + 2 * i]);
        uint32_t hi = __bfloat16_as_ushort(prow[c * 64 + 2 * i + 1]);
        r[i] = lo | (hi << 16);
      }
      tmem_st32(p_tmem + lane_addr_off + c * 32, r);
    }
    tmem_wait_st();
    tc_fence_before();
  }
  __syncthreads();

  if (threadIdx.x == 0) {
    const uint32_t bar = smem_u32(&sh.bar_load);
    if (kMode == 0) {
      mbar_expect_tx(bar, 4 * kPanelBytes);
      tma_load_4d(smem_u32(smem_a), &tmap_a, bar, 0, 0, 0, 0);
      tma_load_4d(smem_u32(smem_a + kPanelBytes), &tmap_a, bar, 64, 0, 0, 0);
    } else {
      mbar_expect_tx(bar, 2 * kPanelBytes);
    }
    tma_load_4d(smem_u32(smem_b), &tmap_b, bar, 0, 0, 0, 0);
    tma_load_4d(smem_u32(smem_b + kPanelBytes), &tmap_b, bar, 64, 0, 0, 0);
    if (mbar_wait(bar, 0, ctx, 1)) {
      tc_fence_after();
      if (kMode == 0) {
        constexpr uint32_t idesc = make_idesc_bf16(128, 128, false, false);
        const uint64_t a0 = make_smem_desc_sw128(smem_u32(smem_a), 16, 1024);
        const uint64_t b0 = make_smem_desc_sw128(smem_u32(smem_b), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // 16 contraction elements = 32 bytes inside the swizzled row; panel 1 starts 16 KB later.
          const uint64_t off = static_cast<uint64_t>(((kk & 3) * 32 + (kk >> 2) * kPanelBytes) >> 4);
          mma_ss(d_tmem, a0 + off, b0 + off, idesc, kk > 0 ? 1u : 0u);
        }
      } else {
        constexpr uint32_t idesc = make_idesc_bf16(128, 128, false, true);
        const uint64_t b0 = make_smem_desc_sw128(smem_u32(smem_b), kPanelBytes, 1024);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // 16 key rows of V = 2 KB; 16 bf16 of P = 8 tensor-memory columns.
          const uint64_t off = static_cast<uint64_t>((kk * 16 * 128) >> 4);
          mma_ts(d_tmem, p_tmem + kk * 8, b0 + off, idesc, kk > 0 ? 1u : 0u);
        }
      }
      mma_commit(smem_u32(&sh.bar_mma));
    }
  }
  __syncwarp();
  if (mbar_wait(smem_u32(&sh.bar_mma), 0, ctx, 2)) {
    tc_fence_after();
    uint32_t r[32];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      tmem_ld32(d_tmem + lane_addr_off + c * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) out[threadIdx.x * kTile + c * 32 + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 256);
}


// Bounded-wait probe: waits on an mbarrier that nothing will ever arrive on.  The wait must give up
// after `budget_ns`, record DEV_ERR_WAIT_TIMEOUT with the site id in the status words and return, leaving
// the context usable.
__global__ void __launch_bounds__(32) wait_timeout_kernel(unsigned long long budget_ns, int site, int* status,
                                                          int* returned) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    mbar_fence_init();
  }
  __syncwarp();
  AbortCtx ctx{&abort_flag, status};
  const bool ok = mbar_wait(smem_u32(&bar), 0, ctx, site, budget_ns);
  if (threadIdx.x == 0) *returned = ok ? 1 : 2;
}

int launch_tile_test(int mode, const void* a, const void* b, float* out, int32_t* status, void* stream) {
  if (a == nullptr || b == nullptr || out == nullptr) return DTB_ERR_NULL;
  if (!device_is_sm100()) return DTB_ERR_ARCH;
  CUtensorMap ta, tb;
  int st = make_tmap_bhsd(&ta, a, 1, 1, kTile, kTile * kTile, kTile * kTile, kTile, kTile);
  if (st != DTB_OK) return st;
  st = make_tmap_bhsd(&tb, b, 1, 1, kTile, kTile * kTile, kTile * kTile, kTile, kTile);
  if (st != DTB_OK) return st;
  const size_t smem = 4 * kPanelBytes + 1024;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (mode == 0) {
    e = cudaFuncSetAttribute(mma_tile_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (!cuda_ok(e, "cudaFuncSetAttribute")) return DTB_ERR_LAUNCH;
    mma_tile_kernel<0><<<1, 128, smem, s>>>(ta, tb, static_cast<const __nv_bfloat16*>(a), out, status);
  } else {
    e = cudaFuncSetAttribute(mma_tile_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (!cuda_ok(e, "cudaFuncSetAttribute")) return DTB_ERR_LAUNCH;
    mma_tile_kernel<1><<<1, 128, smem, s>>>(ta, tb, static_cast<const __nv_bfloat16*>(a), out, status);
  }
  return launch_ok("selftest launch") ? DTB_OK : DTB_ERR_LAUNCH;
}

}  // namespace
}  // namespace dtb

extern "C" int dtb_selftest_tmem_roundtrip(const float* in, float* out, int32_t* status, void* stream) {
  if (in == nullptr || out == nullptr) return DTB_ERR_NULL;
  if (!dtb::device_is_sm100()) return DTB_ERR_ARCH;
  dtb::tmem_roundtrip_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(in, out, status);
  return dtb::launch_ok("selftest launch") ? DTB_OK : DTB_ERR_LAUNCH;
}

extern "C" int dtb_selftest_qk(const void* q, const void* k, float* s_out, int32_t* status, void* stream) {
  return dtb::launch_tile_test(0, q, k, s_out, status, stream);
}

extern "C" int dtb_selftest_pv(const void* p, const void* v, float* o_out, int32_t* status, void* stream) {
  return dtb::launch_tile_test(1, p, v, o_out, status, stream);
}

extern "C" int dtb_selftest_wait_timeout(unsigned long long budget_ns, int site, int32_t* status, int32_t* returned,
                                         void* stream) {
  if (status == nullptr || returned == nullptr) return DTB_ERR_NULL;
  if (budget_ns == 0 || budget_ns > 2000000000ull) return DTB_ERR_SHAPE;
  dtb::wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(budget_ns, site, status, returned);
  return dtb::launch_ok("wait_timeout_kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}
