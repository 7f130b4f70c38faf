// Pre-pass in front of the attention kernel: per-head RMSNorm of q and k, rotary embedding, zeroing of
// padded rows and the [B, S, H, D] -> [B, H, S, D] layout change in one read and one write of each tensor,
// with the per-head row-norm maxima the bounded-logit softmax needs collected on the way.
//
// Half a warp per (tensor, batch, position, head) row of 128 bf16: each lane owns 8 elements.  All
// arithmetic is f32 on the bf16 inputs with one rounding at the end.  HBM-bound: 256 bytes in and 256 bytes
// out per row (the rotary tables and norm weights stay in L2).
#include <algorithm>

#include "host_common.h"
#include "ptx.cuh"

namespace dtb {
namespace {

constexpr int kD = 128;

struct PrepassParams {
  const __nv_bfloat16* in[3];   // q, k, v as [B, S, H, D] (element strides below); v may be null
  int64_t sb[3], ss[3], sh[3];
  __nv_bfloat16* out[3];        // contiguous [B, H, S, D]
  const float* weight[2];       // RMSNorm scale of q and k, [D] (null = ones)
  const float* cos;             // [S, rotary] (null = no rotary embedding)
  const float* sin;
  const int32_t* kv_len;        // [B] or null: rows at or past it are written as zeros
  float* norms;                 // [2 * H] or null: max output row norm per head of q (scaled) and k
  float eps, q_norm_mult;
  int B, S, H, rotary, n_tensors;
};

// Half a warp owns a row: lane l of the half owns elements 8l..8l+7 (one 16-byte access).  A block of 8 warps
// takes 8 consecutive positions of one batch element, one position per warp, and walks the heads eight at a
// time (two rows per warp access, four accesses in flight): a warp reads 1 KB of contiguous [B, S, H, D] input per
// step and the block writes 2 KB of contiguous [B, H, S, D] output per head, and the rotary table row of the
// position is loaded once per warp and reused for every head.  Per-head norm maxima are kept in shared memory
// and flushed once per block.
#ifndef DTB_PREPASS_BLOCKS
#define DTB_PREPASS_BLOCKS 4
#endif
constexpr int kTilePositions = 8;
constexpr int kAccessesInFlight = 4;   // 16-byte loads outstanding per lane (two rows each per warp)

__device__ __forceinline__ void unpack8(const uint4& raw, float (&x)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    x[2 * i] = f.x;
    x[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// The two halves of a bf16 pair as f32 (exact).
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

__global__ void __launch_bounds__(256, DTB_PREPASS_BLOCKS) qk_prepass_kernel(const __grid_constant__ PrepassParams p) {
  extern __shared__ int head_max[];                   // [H] row-norm maxima (as int bits) of this block
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int hl = lane & 15;                           // lane within the half warp
  const int sub = lane >> 4;                          // which of the two rows of a warp access
  const int which = blockIdx.y;                       // 0 = q, 1 = k, 2 = v
  const bool want_norms = which < 2 && p.norms != nullptr;
  const int half_lanes = p.rotary / 16;               // lanes holding one half of the rotated channels
  const bool first = hl < half_lanes;
  const bool second = hl >= half_lanes && hl < 2 * half_lanes;
  const int partner = (lane & 16) | ((first ? hl + half_lanes : hl - half_lanes) & 15);
  const int s_tiles = (p.S + kTilePositions - 1) / kTilePositions;
  const int64_t tiles = static_cast<int64_t>(p.B) * s_tiles;
  if (want_norms) {
    for (int i = threadIdx.x; i < p.H; i += blockDim.x) head_max[i] = 0;
    __syncthreads();
  }
  float wgt[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
  if (which < 2 && p.weight[which] != nullptr) {
    const float4 a = reinterpret_cast<const float4*>(p.weight[which])[2 * hl];
    const float4 c = reinterpret_cast<const float4*>(p.weight[which])[2 * hl + 1];
    wgt[0] = a.x; wgt[1] = a.y; wgt[2] = a.z; wgt[3] = a.w; wgt[4] = c.x; wgt[5] = c.y; wgt[6] = c.z; wgt[7] = c.w;
  }
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int b = static_cast<int>(tile / s_tiles);
    const int s = static_cast<int>(tile % s_tiles) * kTilePositions + warp;
    if (s >= p.S) continue;                           // warp-uniform
    const bool live = p.kv_len == nullptr || s < p.kv_len[b];
    // cos / sin of this lane's eight channels as bf16 pairs (the tables are used in the input dtype, as the
    // reference casts them); lanes outside the rotated channels keep cos = 1, sin = 0
    uint32_t cs2[4], sn2[4];
    if (which < 2 && p.cos != nullptr && (first || second)) {
      const float4* cp = reinterpret_cast<const float4*>(p.cos + static_cast<int64_t>(s) * p.rotary) + 2 * hl;
      const float4* sp = reinterpret_cast<const float4*>(p.sin + static_cast<int64_t>(s) * p.rotary) + 2 * hl;
      const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
      const float sg = first ? -1.0f : 1.0f;   // turned = (-second half, first half)
      cs2[0] = pack_bf16x2(c0.x, c0.y); cs2[1] = pack_bf16x2(c0.z, c0.w);
      cs2[2] = pack_bf16x2(c1.x, c1.y); cs2[3] = pack_bf16x2(c1.z, c1.w);
      sn2[0] = pack_bf16x2(sg * s0.x, sg * s0.y); sn2[1] = pack_bf16x2(sg * s0.z, sg * s0.w);
      sn2[2] = pack_bf16x2(sg * s1.x, sg * s1.y); sn2[3] = pack_bf16x2(sg * s1.z, sg * s1.w);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) { cs2[i] = 0x3f803f80u; sn2[i] = 0u; }
    }
    const __nv_bfloat16* in_row = p.in[which] + b * p.sb[which] + s * p.ss[which];
    __nv_bfloat16* out_row = p.out[which] + (static_cast<int64_t>(b) * p.H * p.S + s) * kD;
    for (int h0 = 0; h0 < p.H; h0 += 2 * kAccessesInFlight) {
      uint4 raw[kAccessesInFlight];
      int hh[kAccessesInFlight];
#pragma unroll
      for (int u = 0; u < kAccessesInFlight; ++u) {
        hh[u] = h0 + 2 * u + sub;
        raw[u] = make_uint4(0u, 0u, 0u, 0u);
        if (live && hh[u] < p.H) raw[u] = reinterpret_cast<const uint4*>(in_row + hh[u] * p.sh[which])[hl];
      }
#pragma unroll
      for (int u = 0; u < kAccessesInFlight; ++u) {
        uint4 packed = raw[u];
        if (which < 2) {
          float x[8];
          unpack8(raw[u], x);
          float ssq = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) ssq += x[i] * x[i];
          ssq = half_warp_sum(ssq);
          const float rrms = rsqrtf(ssq * (1.0f / kD) + p.eps);
          // normalised values, rounded to bf16 as the reference's RMSNorm returns them, kept as bf16 pairs
          uint32_t yp[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            yp[i] = pack_bf16x2(x[2 * i] * rrms * wgt[2 * i], x[2 * i + 1] * rrms * wgt[2 * i + 1]);
          if (p.cos != nullptr) {
            // channel c < rotary/2 pairs with c + rotary/2: out = y*cos + turned*sin; the partner's values
            // travel as the bf16 pairs they already are
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t op = __shfl_sync(0xffffffffu, yp[i], partner);
              const float y0 = bf16_lo(yp[i]) * bf16_lo(cs2[i]) + bf16_lo(op) * bf16_lo(sn2[i]);
              const float y1 = bf16_hi(yp[i]) * bf16_hi(cs2[i]) + bf16_hi(op) * bf16_hi(sn2[i]);
              yp[i] = pack_bf16x2(y0, y1);
            }
          }
          packed = make_uint4(yp[0], yp[1], yp[2], yp[3]);
          if (!live) packed = make_uint4(0u, 0u, 0u, 0u);
          if (want_norms) {
            float z[8];
            unpack8(packed, z);
            float n2 = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) n2 += z[i] * z[i];
            n2 = half_warp_sum(n2);
            if (hl == 0 && live && hh[u] < p.H)
              atomicMax(&head_max[hh[u]], __float_as_int(sqrtf(n2) * (which == 0 ? p.q_norm_mult : 1.0f)));
          }
        }
        if (hh[u] < p.H) reinterpret_cast<uint4*>(out_row + static_cast<int64_t>(hh[u]) * p.S * kD)[hl] = packed;
      }
    }
  }
  if (want_norms) {
    __syncthreads();
    for (int i = threadIdx.x; i < p.H; i += blockDim.x)
      if (head_max[i] != 0) atomicMax(reinterpret_cast<int*>(p.norms + which * p.H + i), head_max[i]);
  }
}

__global__ void prepass_bound_kernel(const float* __restrict__ norms, int H, float gate, float* __restrict__ mk) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  const float bound = norms[h] * norms[H + h];
  mk[h] = ceilf(bound);
  mk[H + h] = (bound <= gate) ? 1.0f : 0.0f;
}

}  // namespace
}  // namespace dtb

extern "C" int dtb_qk_prepass(const dtb_prepass_params* pp, void* stream) {
  using namespace dtb;
  if (pp == nullptr || pp->q_in == nullptr || pp->k_in == nullptr || pp->q_out == nullptr || pp->k_out == nullptr)
    return DTB_ERR_NULL;
  if ((pp->v_in == nullptr) != (pp->v_out == nullptr)) return DTB_ERR_NULL;
  if ((pp->cos == nullptr) != (pp->sin == nullptr)) return DTB_ERR_NULL;
  if (pp->D != kD || pp->B <= 0 || pp->S <= 0 || pp->H <= 0) return DTB_ERR_SHAPE;
  if (pp->cos != nullptr && (pp->rotary <= 0 || pp->rotary > kD || pp->rotary % 16 != 0)) return DTB_ERR_SHAPE;
  if ((pp->mk_out != nullptr) != (pp->norms != nullptr)) return DTB_ERR_NULL;
  PrepassParams kp;
  const void* ins[3] = {pp->q_in, pp->k_in, pp->v_in};
  void* outs[3] = {pp->q_out, pp->k_out, pp->v_out};
  const int64_t* strides[3] = {pp->q_strides, pp->k_strides, pp->v_strides};
  kp.n_tensors = pp->v_in != nullptr ? 3 : 2;
  for (int i = 0; i < 3; ++i) {
    const int u = i < kp.n_tensors ? i : 0;
    if ((reinterpret_cast<uintptr_t>(ins[u]) & 15u) || (reinterpret_cast<uintptr_t>(outs[u]) & 15u)) return DTB_ERR_ALIGN;
    if ((strides[u][0] & 7) || (strides[u][1] & 7) || (strides[u][2] & 7)) return DTB_ERR_ALIGN;
    kp.in[i] = static_cast<const __nv_bfloat16*>(ins[u]);
    kp.out[i] = static_cast<__nv_bfloat16*>(outs[u]);
    kp.sb[i] = strides[u][0];
    kp.ss[i] = strides[u][1];
    kp.sh[i] = strides[u][2];
  }
  if ((reinterpret_cast<uintptr_t>(pp->cos) & 15u) || (reinterpret_cast<uintptr_t>(pp->sin) & 15u) ||
      (reinterpret_cast<uintptr_t>(pp->q_weight) & 15u) || (reinterpret_cast<uintptr_t>(pp->k_weight) & 15u))
    return DTB_ERR_ALIGN;
  kp.weight[0] = pp->q_weight;
  kp.weight[1] = pp->k_weight;
  kp.cos = pp->cos;
  kp.sin = pp->sin;
  kp.kv_len = pp->kv_len;
  kp.norms = pp->norms;
  kp.eps = pp->eps;
  const float scale = pp->scale > 0.f ? pp->scale : 1.0f / sqrtf(static_cast<float>(kD));
  kp.q_norm_mult = scale * 1.44269504f;
  kp.B = pp->B;
  kp.S = pp->S;
  kp.H = pp->H;
  kp.rotary = pp->cos != nullptr ? pp->rotary : 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (pp->norms != nullptr &&
      !cuda_ok(cudaMemsetAsync(pp->norms, 0, sizeof(float) * 2 * pp->H, s), "cudaMemsetAsync(norms)"))
    return DTB_ERR_LAUNCH;
  if (pp->H > 8192) return DTB_ERR_SHAPE;
  const int64_t tiles = static_cast<int64_t>(pp->B) * ((pp->S + 7) / 8);
  const unsigned blocks = static_cast<unsigned>(std::min<int64_t>(tiles, 148 * 8));
  qk_prepass_kernel<<<dim3(blocks, kp.n_tensors), 256, sizeof(int) * pp->H, s>>>(kp);
  if (!launch_ok("qk_prepass_kernel launch")) return DTB_ERR_LAUNCH;
  if (pp->mk_out != nullptr) {
    prepass_bound_kernel<<<(pp->H + 127) / 128, 128, 0, s>>>(pp->norms, pp->H, pp->gate > 0.f ? pp->gate : 213.0f,
                                                             pp->mk_out);
    if (!launch_ok("prepass_bound_kernel launch")) return DTB_ERR_LAUNCH;
  }
  return DTB_OK;
}
