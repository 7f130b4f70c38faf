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

// Tensor-pipe rate probe: one CTA issues `iters` rounds of 8 back-to-back MMAs (one 128-deep
// contraction) on garbage operands and reports the cycles from first issue to completion.
//   mode 0: SS 128x128x16   mode 1: SS 128x64x16   mode 2: TS 128x128x16 (A in tensor memory)
//   mode 3: SS 128x256x16
__global__ void __launch_bounds__(128) mma_rate_kernel(int mode, int iters, long long* out, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ SelftestShared sh;
  uint8_t* smem = align_1024(smem_raw);
  const int warp = threadIdx.x >> 5;
  AbortCtx ctx{&sh.abort_flag, status};
  if (threadIdx.x == 0) {
    sh.abort_flag = 0;
    mbar_init(smem_u32(&sh.bar_mma), 1);
    mbar_init(smem_u32(&sh.bar_mma2), 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&sh.tmem_base), 512);
    tmem_relinquish();
  }
  // finite operands: zero the shared tiles (A 32 KB, B 64 KB)
  for (int i = threadIdx.x; i < (96 * 1024) / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = sh.tmem_base;
  {
    uint32_t z[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) z[i] = 0;
    for (int c = 0; c < 16; ++c) tmem_st32(tbase + (static_cast<uint32_t>(warp * 32) << 16) + c * 32, z);
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  // Modes 0-3: one thread issues eight MMAs per accumulator, alternating between two accumulators.
  // Mode 4: as mode 0, but consecutive instructions alternate accumulators.
  // Mode 5: as mode 0, with a second thread (another warp) issuing the same stream into its own accumulators.
  // Mode 6: consecutive instructions alternate between the shared-memory-A form (accumulator 0) and the
  //         tensor-memory-A form (accumulator 1), the mix an attention iteration issues.
  const bool second_issuer = mode == 5 && threadIdx.x == 32;
  if (threadIdx.x == 0 || second_issuer) {
    tc_fence_after();
    const int n = mode == 1 ? 64 : (mode == 3 ? 256 : 128);
    const uint32_t idesc = make_idesc_bf16(128, n, false, mode == 2);
    const uint32_t idesc_ts = make_idesc_bf16(128, 128, false, true);
    const uint64_t a0 = make_smem_desc_sw128(smem_u32(smem), 16, 1024);
    const uint64_t b0 = mode == 2 ? make_smem_desc_sw128(smem_u32(smem + 32768), kPanelBytes, 1024)
                                  : make_smem_desc_sw128(smem_u32(smem + 32768), 16, 1024);
    const uint64_t bv = make_smem_desc_sw128(smem_u32(smem + 65536), kPanelBytes, 1024);
    const uint32_t acc_base = tbase + (second_issuer ? 128u : 0u);
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
      const uint32_t d = acc_base + ((it & 1) ? 256u : 0u);   // alternate accumulators
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t off = static_cast<uint64_t>(((kk & 3) * 32 + (kk >> 2) * kPanelBytes) >> 4);
        if (mode == 2) {
          mma_ts(d, tbase + 448 + kk * 8, b0 + static_cast<uint64_t>((kk * 2048) >> 4), idesc, 1u);
        } else if (mode == 4) {
          mma_ss(tbase + ((kk & 1) ? 256u : 0u), a0 + off, b0 + off, idesc, 1u);
        } else if (mode == 6) {
          if (kk & 1) mma_ts(tbase + 256u, tbase + 448 + kk * 8, bv + static_cast<uint64_t>((kk * 2048) >> 4), idesc_ts, 1u);
          else mma_ss(tbase, a0 + off, b0 + off, idesc, 1u);
        } else {
          mma_ss(d, a0 + off, b0 + off, idesc, 1u);
        }
      }
    }
    mma_commit(smem_u32(second_issuer ? &sh.bar_mma2 : &sh.bar_mma));
    if (threadIdx.x == 0) {
      const long long t1 = clock64();
      bool ok = mbar_wait(smem_u32(&sh.bar_mma), 0, ctx, 3);
      if (mode == 5 && ok) ok = mbar_wait(smem_u32(&sh.bar_mma2), 0, ctx, 4);
      const long long t2 = clock64();
      out[0] = t1 - t0;
      out[1] = t2 - t0;
      out[2] = ok ? 1 : 0;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 512);
}

// Issue-path probe: the same back-to-back MMA stream as mma_rate_kernel mode kMode (0: SS N=128, 1: SS N=64,
// 2: TS N=128, 3: SS N=256, 4: SS N=128 alternating accumulators per instruction; 5: as 2 with what an attention
// iteration does between blocks of four instructions - an arrive on, a satisfied wait for and a fence after an
// mbarrier; 6: as 2 with the thread idling `gap_cycles` between blocks of four, which shows how many cycles of
// issue-side work the pipe's queue covers; 7: as 2 with only the fence between blocks; 8: only a satisfied
// wait; 9: a satisfied wait and the fence; 10: the barrier poll for a block issued before the previous block's
// instructions and only consumed after them; 11: a volatile shared-memory load and test; 12: a tcgen05.commit
// between blocks; 13: as 2 while the other three warps load and store tensor memory; 14: as 0 with operand
// descriptors that change every block; 15: as 14 carrying only the low descriptor words; 16: as 14 while six
// warps store to shared memory; 17 / 18: as 14 with two arithmetic-bound warps on the issuing warp's / on another
// sub-partition; 19: as 15 with the arithmetic warps of 17), written four ways:
//   kStyle 0: one thread inside a divergent branch, tensor-memory base read from shared memory
//   kStyle 1: as 0, tensor-memory base taken as the constant 0 (checked: the CTA owns all 512 columns)
//   kStyle 2: the whole warp runs the loop and computes the operands; the instruction itself is predicated
//             on lane 0, tensor-memory base read from shared memory
//   kStyle 3: as 2 with the constant base
// The operands of tcgen05.mma live in uniform registers; the styles differ in how much work it takes to
// get them there, which is what bounds the issue rate of a single thread.
template <int kStyle, int kMode>
__global__ void __launch_bounds__(384) mma_issue_kernel(int iters, int gap_cycles, long long* out, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ SelftestShared sh;
  uint8_t* smem = align_1024(smem_raw);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  AbortCtx ctx{&sh.abort_flag, status};
  if (threadIdx.x == 0) {
    sh.abort_flag = 0;
    mbar_init(smem_u32(&sh.bar_mma), 1);
    mbar_init(smem_u32(&sh.bar_load), 1);
    mbar_init(smem_u32(&sh.bar_mma2), 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&sh.tmem_base), 512);
    tmem_relinquish();
  }
  for (int i = threadIdx.x; i < (96 * 1024) / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase_mem = sh.tmem_base;
  if (warp < 4) {
    uint32_t z[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) z[i] = 0;
    for (int c = 0; c < 16; ++c) tmem_st32(tbase_mem + (static_cast<uint32_t>(warp * 32) << 16) + c * 32, z);
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  constexpr bool kConstBase = (kStyle & 1) != 0;
  constexpr bool kWholeWarp = kStyle >= 2;
  if (kMode == 16 && (warp & 3) != 0 && warp < 8) {
    // six warps store into an unused part of shared memory, one 512-byte warp store every gap_cycles each,
    // for about as long as the instruction stream runs: does other shared-memory traffic slow the operand fetch?
    const uint32_t dst = smem_u32(smem + 72 * 1024) + threadIdx.x * 16;
    const long long t_end = clock64() + static_cast<long long>(iters) * 8 * 64;
    uint32_t n = 0;
    while (clock64() < t_end) {
      asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(n) : "memory");
      ++n;
      const long long g0 = clock64();
      while (clock64() - g0 < gap_cycles) {}
    }
  }
  if (((kMode == 17 || kMode == 19) && (warp == 4 || warp == 8)) || (kMode == 18 && (warp == 5 || warp == 9))) {
    // two warps of arithmetic (FMA and ex2, the softmax mix) on the issuing warp's sub-partition (17) or on
    // another one (18): does competing for issue slots slow the instruction stream?
    const long long t_end = clock64() + static_cast<long long>(iters) * 8 * 64;
    float a[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) a[c] = 0.001f * static_cast<float>(threadIdx.x + c);
    // gap_cycles picks the mix: 0 FMA and ex2 (8:1), 16 FMA only, 32 ex2 only, 48 integer multiply-add only,
    // 64 one warp-wide instruction every ~32 cycles (a warp that mostly sleeps)
    const int mix = gap_cycles >> 4;
    uint32_t ia[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) ia[c] = threadIdx.x + c;
    while (clock64() < t_end) {
      if (mix == 0) {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
#pragma unroll
          for (int c = 0; c < 8; ++c) a[c] = fmaf(a[c], 0.999f, 0.001f);
          a[r] = ex2(a[r] - 1.0f);
        }
      } else if (mix == 1) {
#pragma unroll
        for (int r = 0; r < 9; ++r) {
#pragma unroll
          for (int c = 0; c < 8; ++c) a[c] = fmaf(a[c], 0.999f, 0.001f);
        }
      } else if (mix == 2) {
#pragma unroll
        for (int c = 0; c < 8; ++c) a[c] = ex2(a[c] - 1.0f);
      } else if (mix == 3) {
#pragma unroll
        for (int r = 0; r < 9; ++r) {
#pragma unroll
          for (int c = 0; c < 8; ++c) ia[c] = ia[c] * 3u + 7u;
        }
      } else {
        __nanosleep(20);
      }
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) a[c] += __uint_as_float(ia[c] & 0xffu);
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) sum += a[c];
    if (sum == 123.456f) out[2] = 7;   // keep the arithmetic alive
  }
  if (kMode == 13 && warp > 0 && warp < 4) {
    // the other three warps read and write tensor memory the way softmax threads do, for about as long as
    // the instruction stream runs
    tc_fence_after();
    uint32_t r[128];
    uint32_t acc = 0;
    const uint32_t lane_base = tbase_mem + (static_cast<uint32_t>(warp * 32) << 16);
    for (int i = 0; i < iters * 4; ++i) {
      tmem_ld128_sync(lane_base + 128, r);
#pragma unroll
      for (int c = 0; c < 128; ++c) acc += r[c];
      tmem_st32(lane_base + 128, *reinterpret_cast<const uint32_t(*)[32]>(&r[0]));
      tmem_wait_st();
    }
    if (acc == 0x12345678u) out[2] = 7;   // keep the loads alive
  }
  if (kConstBase && tbase_mem != 0) {
    if (threadIdx.x == 0) report_error(ctx, DEV_ERR_WAIT_TIMEOUT, 5, static_cast<int>(tbase_mem));
  } else if (warp == 0 && (kWholeWarp || lane == 0)) {
    tc_fence_after();
    const uint32_t tbase = kConstBase ? 0u : tbase_mem;
    constexpr int n = kMode == 1 ? 64 : (kMode == 3 ? 256 : 128);
    constexpr bool kTs = kMode == 2 || (kMode >= 5 && kMode < 14);
    constexpr uint32_t idesc = make_idesc_bf16(128, n, false, kTs);
    const uint64_t a0 = make_smem_desc_sw128(smem_u32(smem), 16, 1024);
    const uint64_t b0 = kTs ? make_smem_desc_sw128(smem_u32(smem + 32768), kPanelBytes, 1024)
                                   : make_smem_desc_sw128(smem_u32(smem + 32768), 16, 1024);
    const uint32_t issue = kWholeWarp ? (lane == 0 ? 1u : 0u) : 1u;
    bool polled = kMode == 10 ? mbar_test_wait(smem_u32(&sh.bar_mma2), 1) : false;
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
      const uint32_t d = tbase + ((it & 1) ? 256u : 0u);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t off = static_cast<uint64_t>(((kk & 3) * 32 + (kk >> 2) * kPanelBytes) >> 4);
        if (kMode >= 14) {
          // operands that change from block to block, as in an attention iteration: the B tile moves through
          // four slots and the A tile alternates
          // (shifts of whole 1024-byte swizzle atoms; the furthest byte read stays below 68 KB of the 96 KB)
          const uint32_t a_byte = ((it >> 1) & 1) * 1024u;
          const uint32_t b_byte = (it & 3) * 1024u;
          if (kMode != 15 && kMode != 19) {
            mma_ss_if(issue, d, a0 + static_cast<uint64_t>(a_byte >> 4) + off, b0 + static_cast<uint64_t>(b_byte >> 4) + off, idesc, 1u);
          } else {
            mma_ss_lo(d, static_cast<uint32_t>(a0) + (a_byte >> 4) + static_cast<uint32_t>(off),
                      static_cast<uint32_t>(b0) + (b_byte >> 4) + static_cast<uint32_t>(off), idesc, 1u, issue);
          }
          continue;
        }
        if (kMode >= 5 && (kk & 3) == 0 && issue) {
          if (kMode == 12 || kMode == 13) {
            if (kMode == 12 && it + kk > 0) mma_commit(smem_u32(&sh.bar_load));
          } else if (kMode == 10) {
            // the poll for this block was issued before the previous block's instructions
            if (!polled && !mbar_wait(smem_u32(&sh.bar_mma2), 1, ctx, 8)) break;
            tc_fence_after();
            polled = mbar_test_wait(smem_u32(&sh.bar_mma2), 1);
          } else if (kMode == 11) {
            if (*reinterpret_cast<volatile int*>(&sh.abort_flag) != 0) break;
          } else if (kMode == 7) {
            tc_fence_after();
          } else if (kMode == 8 || kMode == 9) {
            // parity 1 of a barrier still in its first phase: the wait is satisfied at once
            if (!mbar_wait(smem_u32(&sh.bar_mma2), 1, ctx, 7)) break;
            if (kMode == 9) tc_fence_after();
          } else if (kMode == 5) {
            const uint32_t bar = smem_u32(&sh.bar_load);
            const uint32_t phase = static_cast<uint32_t>(it * 2 + (kk >> 2)) & 1u;
            mbar_arrive(bar);
            if (!mbar_wait(bar, phase, ctx, 6)) break;
            tc_fence_after();
          } else {
            const long long g0 = clock64();
            while (clock64() - g0 < gap_cycles) {}
          }
        }
        if (kTs) {
          mma_ts_if(issue, d, tbase + 448 + kk * 8, b0 + static_cast<uint64_t>((kk * 2048) >> 4), idesc, 1u);
        } else if (kMode == 4) {
          mma_ss_if(issue, tbase + ((kk & 1) ? 256u : 0u), a0 + off, b0 + off, idesc, 1u);
        } else {
          mma_ss_if(issue, d, a0 + off, b0 + off, idesc, 1u);
        }
      }
    }
    if (issue) mma_commit(smem_u32(&sh.bar_mma));
    __syncwarp(kWholeWarp ? 0xffffffffu : 1u);
    const long long t1 = clock64();
    const bool ok = mbar_wait(smem_u32(&sh.bar_mma), 0, ctx, 3);
    const long long t2 = clock64();
    if (lane == 0) {
      out[0] = t1 - t0;
      out[1] = t2 - t0;
      out[2] = ok ? 1 : 0;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase_mem, 512);
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

namespace {
template <int kStyle, int kMode>
int launch_issue_probe(int iters, int gap, long long* out, int32_t* status, cudaStream_t stream) {
  const size_t smem = 96 * 1024 + 1024;
  if (!dtb::cuda_ok(cudaFuncSetAttribute(dtb::mma_issue_kernel<kStyle, kMode>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem), "cudaFuncSetAttribute"))
    return DTB_ERR_LAUNCH;
  dtb::mma_issue_kernel<kStyle, kMode><<<1, 384, smem, stream>>>(iters, gap, out, status);
  return dtb::launch_ok("mma_issue_kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}
template <int kStyle>
int launch_issue_style(int base, int iters, int gap, long long* out, int32_t* status, cudaStream_t stream) {
  switch (base) {
    case 0: return launch_issue_probe<kStyle, 0>(iters, gap, out, status, stream);
    case 1: return launch_issue_probe<kStyle, 1>(iters, gap, out, status, stream);
    case 2: return launch_issue_probe<kStyle, 2>(iters, gap, out, status, stream);
    case 3: return launch_issue_probe<kStyle, 3>(iters, gap, out, status, stream);
    case 4: return launch_issue_probe<kStyle, 4>(iters, gap, out, status, stream);
    case 5: return launch_issue_probe<kStyle, 5>(iters, gap, out, status, stream);
    case 6: return launch_issue_probe<kStyle, 6>(iters, gap, out, status, stream);
    case 7: return launch_issue_probe<kStyle, 7>(iters, gap, out, status, stream);
    case 8: return launch_issue_probe<kStyle, 8>(iters, gap, out, status, stream);
    case 9: return launch_issue_probe<kStyle, 9>(iters, gap, out, status, stream);
    case 10: return launch_issue_probe<kStyle, 10>(iters, gap, out, status, stream);
    case 11: return launch_issue_probe<kStyle, 11>(iters, gap, out, status, stream);
    case 12: return launch_issue_probe<kStyle, 12>(iters, gap, out, status, stream);
    case 13: return launch_issue_probe<kStyle, 13>(iters, gap, out, status, stream);
    case 14: return launch_issue_probe<kStyle, 14>(iters, gap, out, status, stream);
    case 15: return launch_issue_probe<kStyle, 15>(iters, gap, out, status, stream);
    case 16: return launch_issue_probe<kStyle, 16>(iters, gap, out, status, stream);
    case 17: return launch_issue_probe<kStyle, 17>(iters, gap, out, status, stream);
    case 18: return launch_issue_probe<kStyle, 18>(iters, gap, out, status, stream);
    case 19: return launch_issue_probe<kStyle, 19>(iters, gap, out, status, stream);
    default: return DTB_ERR_SHAPE;
  }
}
}  // namespace

extern "C" int dtb_selftest_mma_rate(int mode, int iters, long long* out_cycles, int32_t* status, void* stream) {
  if (out_cycles == nullptr) return DTB_ERR_NULL;
  if (mode < 0 || iters <= 0 || iters > 100000) return DTB_ERR_SHAPE;
  if (!dtb::device_is_sm100()) return DTB_ERR_ARCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (mode >= 100) {   // 1000 * gap / 16 + 100 + 20 * style + stream shape: the issue-path probe
    const int gap = (mode / 1000) * 16;
    mode %= 1000;
    if (mode < 100) return DTB_ERR_SHAPE;
    const int style = (mode - 100) / 20, base = (mode - 100) % 20;
    switch (style) {
      case 0: return launch_issue_style<0>(base, iters, gap, out_cycles, status, st);
      case 1: return launch_issue_style<1>(base, iters, gap, out_cycles, status, st);
      case 2: return launch_issue_style<2>(base, iters, gap, out_cycles, status, st);
      case 3: return launch_issue_style<3>(base, iters, gap, out_cycles, status, st);
      default: return DTB_ERR_SHAPE;
    }
  }
  if (mode > 6) return DTB_ERR_SHAPE;
  const size_t smem = 96 * 1024 + 1024;
  if (!dtb::cuda_ok(cudaFuncSetAttribute(dtb::mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                    "cudaFuncSetAttribute"))
    return DTB_ERR_LAUNCH;
  dtb::mma_rate_kernel<<<1, 128, smem, st>>>(mode, iters, out_cycles, status);
  return dtb::launch_ok("mma_rate_kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}

extern "C" int dtb_selftest_wait_timeout(unsigned long long budget_ns, int site, int32_t* status, int32_t* returned,
                                         void* stream) {
  if (status == nullptr || returned == nullptr) return DTB_ERR_NULL;
  if (budget_ns == 0 || budget_ns > 2000000000ull) return DTB_ERR_SHAPE;
  dtb::wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(budget_ns, site, status, returned);
  return dtb::launch_ok("wait_timeout_kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}
