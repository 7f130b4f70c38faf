// Output projection behind head-sharded attention output ("keep heads"): the step after the attention call in a
// DiT block whose attention output stays split by heads.  `to_out` contracts over the heads, so each GPU multiplies
// its own heads' output by its rows of the weight and the partial sums of the GPUs are added
// (diffusers_tpu/models/minimax_h3/jax_image_pipeline.py:574-593: "its partial sums meet in one all-reduce").
//
//   y[b, s, :] (+)= sum over local heads h of  o[b, h, s, :] . w[h * 128 : (h + 1) * 128, :]
//
// One CTA per 128 x 256 output tile, two CTAs per SM (one's epilogue runs under the other's main loop); the
// contraction runs over (head, 64-channel half) chunks.  Measured against 128 x 128 tiles with three ring slots
// (1090 TFLOP/s) and 128 x 256 with four slots and one CTA per SM (1215): 1250 TFLOP/s on the C2 / C3 shapes.  The attention
// output is read in place in its [B, H, S, D] layout (the head index is one coordinate of the TMA box, so no
// heads -> channels transpose is ever materialised).  192 threads:
//   warp 0      TMA producer: A chunk 128 rows x 64 channels of one head, W chunk 64 x 256, 2-slot ring
//   warp 1      MMA issuer: tcgen05.mma kind::f16, A K-major and W MN-major from shared memory, f32 in tensor memory
//   warps 2-5   epilogue: tensor memory -> registers -> bf16 rows of y; or, for the reduce-scatter over head shards,
//               straight to the GPU that owns those rows (this one or a peer over NVLink): either bf16 partial rows
//               stored into that GPU's staging slot for this rank (summed there by sum_partials_kernel), so the
//               transfer runs under the GEMM tile by tile, or f32 vector reductions (red.add) into its accumulation
//               buffer.  No TMA or multicast touches peer memory: plain stores and reductions only.
// Bound: tensor cores (arithmetic intensity ~ N / 2 FLOP per byte of o at fixed w); with the reduction fused the
// call is bound by the f32 partial sums crossing NVLink (4 bytes per output element per contributing GPU).
#include <algorithm>
#include <atomic>

#include "host_common.h"
#include "ptx.cuh"

namespace dtb {
namespace {

#ifndef DTB_PROJ_TILE_N
#define DTB_PROJ_TILE_N 256
#define DTB_PROJ_STAGES 2
#define DTB_PROJ_CTAS_PER_SM 2
#endif
constexpr int kTileM = 128;
constexpr int kTileN = DTB_PROJ_TILE_N;
constexpr int kChunkK = 64;
constexpr int kProjStages = DTB_PROJ_STAGES;
constexpr uint32_t kABytes = kTileM * kChunkK * 2;      // 16 KB
constexpr uint32_t kWPanelBytes = kChunkK * 64 * 2;     // 8 KB: 64 contraction rows x 64 output columns
constexpr uint32_t kWBytes = (kTileN / 64) * kWPanelBytes;
constexpr uint32_t kStageBytes = kABytes + kWBytes;
constexpr int kProjThreads = 192;

struct __align__(8) ProjBarriers {
  uint64_t full[kProjStages];
  uint64_t empty[kProjStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

constexpr size_t kProjSmemBytes = 1024 + kProjStages * kStageBytes + sizeof(ProjBarriers);
static_assert(kTileN == 256, "the staged epilogue writes 32 lanes x 8 columns per row");
static_assert(kProjStages * kStageBytes >= 4 * 32 * kTileN * 2, "the epilogue stages its rows in the pipeline slots");

struct ProjParams {
  CUtensorMap tmap_o, tmap_w;
  __nv_bfloat16* out;            // store mode: bf16 [B, S, N]
  int64_t out_stride_b, out_stride_s;
  void* red_dst[8];              // n_dest > 0: per destination f32 [rows_per_dest, N] (reductions) or
  int n_dest, rows_per_dest;     //             bf16 [n_src, rows_per_dest, N] (partials stored at slot src_rank)
  int partials, src_rank;
  int B, Hl, S, N;
  int32_t* status;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* tmap, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst_smem), "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void red_add_v4(float* dst, float a, float b, float c, float d) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

__global__ void __launch_bounds__(kProjThreads, DTB_PROJ_CTAS_PER_SM) out_proj_kernel(const __grid_constant__ ProjParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem;
  {
    const uint32_t a = smem_u32(smem_raw);
    smem = smem_raw + (((a + 1023u) & ~1023u) - a);
  }
  ProjBarriers* bars = reinterpret_cast<ProjBarriers*>(smem + kProjStages * kStageBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kTileN;
  const int m0 = blockIdx.y * kTileM;
  const int b = blockIdx.z;
  const int chunks = p.Hl * 2;               // contraction chunks of 64: (head, channel half)
  AbortCtx ctx{&bars->abort_flag, p.status};

  if (threadIdx.x == 0) {
    bars->abort_flag = 0;
    for (int i = 0; i < kProjStages; ++i) {
      mbar_init(smem_u32(&bars->full[i]), 1);
      mbar_init(smem_u32(&bars->empty[i]), 1);
    }
    mbar_init(smem_u32(&bars->acc_full), 1);
    mbar_fence_init();
    tma_prefetch_desc(&p.tmap_o);
    tma_prefetch_desc(&p.tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars->tmem_base), kTileN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      for (int kc = 0; kc < chunks && ok; ++kc) {
        const int slot = kc % kProjStages;
        const int use = kc / kProjStages;
        if (use > 0) ok = mbar_wait(smem_u32(&bars->empty[slot]), (use - 1) & 1, ctx, 30 + slot);
        if (!ok) break;
        const uint32_t bar = smem_u32(&bars->full[slot]);
        mbar_expect_tx(bar, kStageBytes);
        const uint32_t dst = smem_u32(smem + slot * kStageBytes);
        tma_load_4d(dst, &p.tmap_o, bar, (kc & 1) * kChunkK, m0, kc >> 1, b);
#pragma unroll
        for (int pn = 0; pn < kTileN / 64; ++pn)
          tma_load_2d(dst + kABytes + pn * kWPanelBytes, &p.tmap_w, bar, n0 + 64 * pn, kc * kChunkK);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc_bf16(kTileM, kTileN, false, true);
    bool ok = true;
    for (int kc = 0; kc < chunks && ok; ++kc) {
      const int slot = kc % kProjStages;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->full[slot]), (kc / kProjStages) & 1, ctx, 20 + slot));
      if (!ok) break;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t base = smem_u32(smem + slot * kStageBytes);
        const uint64_t a_desc = make_smem_desc_sw128(base, 16, 1024);
        const uint64_t w_desc = make_smem_desc_sw128(base + kABytes, kWPanelBytes, 1024);
#pragma unroll
        for (int kk = 0; kk < kChunkK / 16; ++kk) {
          mma_ss(tmem_base, a_desc + static_cast<uint64_t>((kk * 32) >> 4), w_desc + static_cast<uint64_t>((kk * 16 * 128) >> 4),
                 idesc, (kc > 0 || kk > 0) ? 1u : 0u);
        }
        mma_commit(smem_u32(&bars->empty[slot]));
        if (kc + 1 == chunks) mma_commit(smem_u32(&bars->acc_full));
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2-5)
    const int quarter = warp & 3;                     // tensor-memory lane quarter this warp may read
    const int s = m0 + quarter * 32 + lane;           // sequence position of this thread's row
    const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->acc_full), 0, ctx, 40));
    if (ok) {
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      const bool live = s < p.S;
      float* red_row = nullptr;
      __nv_bfloat16* out_row = nullptr;
      if (live) {
        if (p.n_dest > 0) {
          const int64_t g = static_cast<int64_t>(b) * p.S + s;       // row of the flattened [B * S, N] result
          const int dest = static_cast<int>(g / p.rows_per_dest);
          const int64_t local = g - static_cast<int64_t>(dest) * p.rows_per_dest;
          if (p.partials)
            out_row = static_cast<__nv_bfloat16*>(p.red_dst[dest]) +
                      (static_cast<int64_t>(p.src_rank) * p.rows_per_dest + local) * p.N;
          else
            red_row = static_cast<float*>(p.red_dst[dest]) + local * p.N;
        } else {
          out_row = p.out + b * p.out_stride_b + s * p.out_stride_s;
        }
      }
      if (p.n_dest > 0 && !p.partials) {
        // f32 reductions straight from registers (each lane owns a row)
#pragma unroll 1
        for (int c = 0; c < kTileN / 32; ++c) {
          uint32_t r[32];
          __syncwarp();                                   // the load is warp-collective: rejoin after the branch
          tmem_ld32_sync(taddr + c * 32, r);
          const int col0 = n0 + c * 32;
          if (!live || col0 >= p.N) continue;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (col0 + 4 * i < p.N)
              red_add_v4(red_row + col0 + 4 * i, __uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                         __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
          }
        }
      } else {
        // bf16 rows: staged in this warp's share of the (now idle) pipeline slots, 16-byte chunks XOR-swizzled by
        // row, then written out a whole 512-byte row per store instruction - full lines for HBM and for NVLink
        uint8_t* stage = smem + quarter * (32 * kTileN * 2);
#pragma unroll 1
        for (int c = 0; c < kTileN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32_sync(taddr + c * 32, r);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1]));
            v.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
            v.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
            v.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
            const int chunk = c * 4 + i;                                         // 16-byte chunk of the row
            *reinterpret_cast<uint4*>(stage + lane * (kTileN * 2) + ((chunk ^ (lane & (kTileN / 8 - 1))) << 4)) = v;
          }
        }
        __syncwarp();
        const int col = n0 + lane * 8;                   // this lane's 8 columns of every row (kTileN == 256)
#pragma unroll 4
        for (int rr = 0; rr < 32; ++rr) {
          const int64_t rp = __shfl_sync(0xffffffffu, reinterpret_cast<int64_t>(out_row), rr);   // row rr's address
          if (rp != 0 && col < p.N) {
            const uint4 v = *reinterpret_cast<const uint4*>(stage + rr * (kTileN * 2) + ((lane ^ (rr & (kTileN / 8 - 1))) << 4));
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(rp) + col) = v;
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (bars->abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem_base, kTileN);
}

// Sum of the bf16 partial projections the ranks stored into this rank's staging buffer [n_src, rows, N]: f32
// accumulation in source order, bf16 result.  8 elements per thread; HBM-bound ((n_src + 1) * rows * N * 2 bytes).
__global__ void __launch_bounds__(256) sum_partials_kernel(const __nv_bfloat16* __restrict__ staged, int n_src,
                                                           int64_t elems, __nv_bfloat16* __restrict__ out) {
  const int64_t chunks = elems / 8;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < chunks;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < n_src; ++r) {
      const uint4 raw = reinterpret_cast<const uint4*>(staged + r * elems)[idx];
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    }
    uint4 v;
    v.x = pack_bf16x2(acc[0], acc[1]);
    v.y = pack_bf16x2(acc[2], acc[3]);
    v.z = pack_bf16x2(acc[4], acc[5]);
    v.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[idx] = v;
  }
}

}  // namespace
}  // namespace dtb

extern "C" int dtb_sum_partials(const void* staged, int32_t n_src, int64_t rows, int32_t N, void* out, void* stream) {
  using namespace dtb;
  if (staged == nullptr || out == nullptr) return DTB_ERR_NULL;
  if (n_src < 1 || n_src > 8 || rows <= 0 || N <= 0 || N % 8 != 0) return DTB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(staged) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u)) return DTB_ERR_ALIGN;
  const int64_t elems = rows * N;
  const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((elems / 8 + 255) / 256, 148 * 16));
  sum_partials_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(staged), n_src, elems, static_cast<__nv_bfloat16*>(out));
  return launch_ok("sum_partials_kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}

extern "C" int dtb_out_proj(const dtb_out_proj_params* pp, void* stream) {
  using namespace dtb;
  if (pp == nullptr || pp->o == nullptr || pp->w == nullptr) return DTB_ERR_NULL;
  if (pp->D != 128 || pp->B <= 0 || pp->H_local <= 0 || pp->S <= 0 || pp->N <= 0 || pp->N % 8 != 0) return DTB_ERR_SHAPE;
  if (pp->B > 65535 || (pp->S + kTileM - 1) / kTileM > 65535) return DTB_ERR_SHAPE;
  if (pp->n_dest < 0 || pp->n_dest > 8) return DTB_ERR_SHAPE;
  if (pp->partials && (pp->n_dest == 0 || pp->src_rank < 0 || pp->src_rank >= 8)) return DTB_ERR_SHAPE;
  ProjParams kp;
  if (pp->n_dest > 0) {
    if (pp->rows_per_dest <= 0 ||
        static_cast<int64_t>(pp->rows_per_dest) * pp->n_dest < static_cast<int64_t>(pp->B) * pp->S)
      return DTB_ERR_SHAPE;
    for (int i = 0; i < pp->n_dest; ++i) {
      if (pp->red_dst[i] == nullptr) return DTB_ERR_NULL;
      if (reinterpret_cast<uintptr_t>(pp->red_dst[i]) & 15u) return DTB_ERR_ALIGN;
    }
    if (pp->N % 8 != 0) return DTB_ERR_ALIGN;
  } else {
    if (pp->out == nullptr) return DTB_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(pp->out) & 15u) || (pp->out_stride_s & 7) || (pp->B > 1 && (pp->out_stride_b & 7)))
      return DTB_ERR_ALIGN;
    if (pp->out_stride_s < pp->N) return DTB_ERR_SHAPE;
  }
  if (pp->w_stride_k < pp->N) return DTB_ERR_SHAPE;
  if (!device_is_sm100()) return DTB_ERR_ARCH;
  int st = make_tmap_bhsd(&kp.tmap_o, pp->o, pp->B, pp->H_local, pp->S, pp->o_stride_b, pp->o_stride_h, pp->o_stride_s,
                          kTileM);
  if (st != DTB_OK) return st;
  st = make_tmap_rows_bf16(&kp.tmap_w, pp->w, static_cast<int64_t>(pp->H_local) * 128, pp->N, pp->w_stride_k, kChunkK, 64);
  if (st != DTB_OK) return st;
  kp.out = static_cast<__nv_bfloat16*>(pp->out);
  kp.out_stride_b = pp->out_stride_b;
  kp.out_stride_s = pp->out_stride_s;
  for (int i = 0; i < 8; ++i) kp.red_dst[i] = i < pp->n_dest ? pp->red_dst[i] : nullptr;
  kp.n_dest = pp->n_dest;
  kp.rows_per_dest = pp->rows_per_dest;
  kp.partials = pp->partials ? 1 : 0;
  kp.src_rank = pp->src_rank;
  kp.B = pp->B;
  kp.Hl = pp->H_local;
  kp.S = pp->S;
  kp.N = pp->N;
  kp.status = pp->status;
  static std::atomic<bool> attr_set[64];      // the opt-in shared-memory size is a per-device function attribute
  int dev = 0;
  if (!cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return DTB_ERR_LAUNCH;
  if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
    if (!cuda_ok(cudaFuncSetAttribute(out_proj_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(kProjSmemBytes)),
                 "out_proj_kernel attributes"))
      return DTB_ERR_LAUNCH;
    if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
  }
  const dim3 grid((pp->N + kTileN - 1) / kTileN, (pp->S + kTileM - 1) / kTileM, pp->B);
  out_proj_kernel<<<grid, kProjThreads, kProjSmemBytes, static_cast<cudaStream_t>(stream)>>>(kp);
  return launch_ok("out_proj_kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}
