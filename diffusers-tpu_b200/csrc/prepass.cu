// Pre-pass in front of the attention kernel: per-head RMSNorm of q and k, rotary embedding, zeroing of
// padded rows and the [B, S, H, D] -> [B, H, S, D] layout change in one read and one write of each tensor,
// with the per-head row-norm maxima the bounded-logit softmax needs collected on the way.
//
// One warp per (tensor, batch, position, head) row of 128 bf16: lane l owns elements 4l..4l+3.  All
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

__global__ void __launch_bounds__(256) qk_prepass_kernel(const __grid_constant__ PrepassParams p) {
  const int lane = threadIdx.x & 31;
  const int which = blockIdx.y;                       // 0 = q, 1 = k, 2 = v
  const int64_t rows = static_cast<int64_t>(p.B) * p.H * p.S;
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * 8;
  const int half_lanes = p.rotary / 8;                // lanes holding one half of the rotated channels
  float best = 0.f;
  int best_h = -1;
  float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
  if (which < 2 && p.weight[which] != nullptr) w = reinterpret_cast<const float4*>(p.weight[which])[lane];
  // rows are visited in output order (b, h, s): a warp mostly stays inside one head
  for (int64_t rid = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); rid < rows; rid += warps_total) {
    const int s = static_cast<int>(rid % p.S);
    const int h = static_cast<int>((rid / p.S) % p.H);
    const int b = static_cast<int>(rid / (static_cast<int64_t>(p.S) * p.H));
    if (which < 2 && p.norms != nullptr && h != best_h) {
      if (best_h >= 0 && lane == 0) atomicMax(reinterpret_cast<int*>(p.norms + which * p.H + best_h), __float_as_int(best));
      best_h = h;
      best = 0.f;
    }
    uint2 packed = make_uint2(0u, 0u);
    const bool padded = p.kv_len != nullptr && s >= p.kv_len[b];
    if (!padded) {
      const uint2 raw = reinterpret_cast<const uint2*>(p.in[which] + b * p.sb[which] + s * p.ss[which] + h * p.sh[which])[lane];
      if (which == 2) {
        packed = raw;
      } else {
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        float x[4] = {lo.x, lo.y, hi.x, hi.y};
        float ssq = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
        const float rrms = rsqrtf(ssq * (1.0f / kD) + p.eps);
        // normalised value, rounded to bf16 as the reference's RMSNorm returns it
        float y[4] = {__bfloat162float(__float2bfloat16(x[0] * rrms * w.x)), __bfloat162float(__float2bfloat16(x[1] * rrms * w.y)),
                      __bfloat162float(__float2bfloat16(x[2] * rrms * w.z)), __bfloat162float(__float2bfloat16(x[3] * rrms * w.w))};
        if (p.cos != nullptr) {
          // channel c < rotary/2 pairs with c + rotary/2: out = y*cos + turned*sin, turned = (-second half, first half)
          const int first = lane < half_lanes;
          const int second = lane >= half_lanes && lane < 2 * half_lanes;
          const int partner = first ? lane + half_lanes : lane - half_lanes;
          float other[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) other[i] = __shfl_sync(0xffffffffu, y[i], partner & 31);
          if (first || second) {
            const float4 c4 = reinterpret_cast<const float4*>(p.cos + static_cast<int64_t>(s) * p.rotary)[lane];
            const float4 s4 = reinterpret_cast<const float4*>(p.sin + static_cast<int64_t>(s) * p.rotary)[lane];
            const float cs[4] = {c4.x, c4.y, c4.z, c4.w};
            const float sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float cb = __bfloat162float(__float2bfloat16(cs[i]));   // tables are used in the input dtype
              const float sb_ = __bfloat162float(__float2bfloat16(sn[i]));
              const float turned = first ? -other[i] : other[i];
              y[i] = y[i] * cb + turned * sb_;
            }
          }
        }
        packed.x = pack_bf16x2(y[0], y[1]);
        packed.y = pack_bf16x2(y[2], y[3]);
        if (p.norms != nullptr) {
          const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&packed.x));
          const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&packed.y));
          float n2 = a.x * a.x + a.y * a.y + c.x * c.x + c.y * c.y;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) n2 += __shfl_xor_sync(0xffffffffu, n2, o);
          best = fmaxf(best, sqrtf(n2) * (which == 0 ? p.q_norm_mult : 1.0f));
        }
      }
    }
    reinterpret_cast<uint2*>(p.out[which] + rid * kD)[lane] = packed;
  }
  if (which < 2 && p.norms != nullptr && best_h >= 0 && lane == 0)
    atomicMax(reinterpret_cast<int*>(p.norms + which * p.H + best_h), __float_as_int(best));
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
  if (pp->cos != nullptr && (pp->rotary <= 0 || pp->rotary > kD || pp->rotary % 8 != 0)) return DTB_ERR_SHAPE;
  if ((pp->mk_out != nullptr) != (pp->norms != nullptr)) return DTB_ERR_NULL;
  PrepassParams kp;
  const void* ins[3] = {pp->q_in, pp->k_in, pp->v_in};
  void* outs[3] = {pp->q_out, pp->k_out, pp->v_out};
  const int64_t* strides[3] = {pp->q_strides, pp->k_strides, pp->v_strides};
  kp.n_tensors = pp->v_in != nullptr ? 3 : 2;
  for (int i = 0; i < 3; ++i) {
    const int u = i < kp.n_tensors ? i : 0;
    if ((reinterpret_cast<uintptr_t>(ins[u]) & 7u) || (reinterpret_cast<uintptr_t>(outs[u]) & 7u)) return DTB_ERR_ALIGN;
    if ((strides[u][0] & 3) || (strides[u][1] & 3) || (strides[u][2] & 3)) return DTB_ERR_ALIGN;
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
  const int64_t rows = static_cast<int64_t>(pp->B) * pp->H * pp->S;
  const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((rows + 7) / 8, 148 * 16));
  qk_prepass_kernel<<<dim3(blocks, kp.n_tensors), 256, 0, s>>>(kp);
  if (!launch_ok("qk_prepass_kernel launch")) return DTB_ERR_LAUNCH;
  if (pp->mk_out != nullptr) {
    prepass_bound_kernel<<<(pp->H + 127) / 128, 128, 0, s>>>(pp->norms, pp->H, pp->gate > 0.f ? pp->gate : 213.0f,
                                                             pp->mk_out);
    if (!launch_ok("prepass_bound_kernel launch")) return DTB_ERR_LAUNCH;
  }
  return DTB_OK;
}
