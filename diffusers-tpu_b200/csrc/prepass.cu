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

// Half a warp owns a row: lane l of the half owns elements 8l..8l+7 (one 16-byte access).  A warp works on
// kRowsInFlight rows at a time so that several independent 256-byte reads are outstanding per warp.
constexpr int kRowsInFlight = 4;

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

__global__ void __launch_bounds__(256) qk_prepass_kernel(const __grid_constant__ PrepassParams p) {
  const int lane = threadIdx.x & 31;
  const int hl = lane & 15;                           // lane within the half warp
  const int sub = lane >> 4;                          // which of the two rows of a warp access
  const int which = blockIdx.y;                       // 0 = q, 1 = k, 2 = v
  const int64_t rows = static_cast<int64_t>(p.B) * p.H * p.S;
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * 8;
  const int half_lanes = p.rotary / 16;               // lanes holding one half of the rotated channels
  float best = 0.f;
  int best_h = -1;
  float wgt[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
  if (which < 2 && p.weight[which] != nullptr) {
    const float4 a = reinterpret_cast<const float4*>(p.weight[which])[2 * hl];
    const float4 c = reinterpret_cast<const float4*>(p.weight[which])[2 * hl + 1];
    wgt[0] = a.x; wgt[1] = a.y; wgt[2] = a.z; wgt[3] = a.w; wgt[4] = c.x; wgt[5] = c.y; wgt[6] = c.z; wgt[7] = c.w;
  }
  // rows are visited in output order (b, h, s): a warp mostly stays inside one head
  for (int64_t base = (static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5)) * kRowsInFlight; base < rows;
       base += warps_total * kRowsInFlight) {
    uint4 raw[kRowsInFlight / 2];
    bool live[kRowsInFlight / 2];
    int hh[kRowsInFlight / 2], ss[kRowsInFlight / 2];
#pragma unroll
    for (int u = 0; u < kRowsInFlight / 2; ++u) {
      const int64_t rid = base + 2 * u + sub;
      const bool in = rid < rows;
      const int64_t r = in ? rid : 0;
      const int s = static_cast<int>(r % p.S);
      const int h = static_cast<int>((r / p.S) % p.H);
      const int b = static_cast<int>(r / (static_cast<int64_t>(p.S) * p.H));
      hh[u] = h;
      ss[u] = s;
      live[u] = in && !(p.kv_len != nullptr && s >= p.kv_len[b]);
      raw[u] = make_uint4(0u, 0u, 0u, 0u);
      if (live[u])
        raw[u] = reinterpret_cast<const uint4*>(p.in[which] + b * p.sb[which] + s * p.ss[which] + h * p.sh[which])[hl];
    }
#pragma unroll
    for (int u = 0; u < kRowsInFlight / 2; ++u) {
      const int64_t rid = base + 2 * u + sub;
      uint4 packed = raw[u];
      if (which < 2) {
        float x[8];
        unpack8(raw[u], x);
        float ssq = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ssq += x[i] * x[i];
        ssq = half_warp_sum(ssq);
        const float rrms = rsqrtf(ssq * (1.0f / kD) + p.eps);
        float y[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)   // normalised value, rounded to bf16 as the reference's RMSNorm returns it
          y[i] = __bfloat162float(__float2bfloat16(x[i] * rrms * wgt[i]));
        if (p.cos != nullptr) {
          // channel c < rotary/2 pairs with c + rotary/2: out = y*cos + turned*sin, turned = (-second half, first half)
          const bool first = hl < half_lanes;
          const bool second = hl >= half_lanes && hl < 2 * half_lanes;
          const int partner = (first ? hl + half_lanes : hl - half_lanes) & 15;
          float other[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) other[i] = __shfl_sync(0xffffffffu, y[i], (lane & 16) | partner);
          if ((first || second) && live[u]) {
            const float4* cp = reinterpret_cast<const float4*>(p.cos + static_cast<int64_t>(ss[u]) * p.rotary) + 2 * hl;
            const float4* sp = reinterpret_cast<const float4*>(p.sin + static_cast<int64_t>(ss[u]) * p.rotary) + 2 * hl;
            const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
            const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float cb = __bfloat162float(__float2bfloat16(cs[i]));   // tables are used in the input dtype
              const float sb_ = __bfloat162float(__float2bfloat16(sn[i]));
              y[i] = y[i] * cb + (first ? -other[i] : other[i]) * sb_;
            }
          }
        }
        packed.x = pack_bf16x2(y[0], y[1]);
        packed.y = pack_bf16x2(y[2], y[3]);
        packed.z = pack_bf16x2(y[4], y[5]);
        packed.w = pack_bf16x2(y[6], y[7]);
        if (!live[u]) packed = make_uint4(0u, 0u, 0u, 0u);
        if (p.norms != nullptr) {
          float z[8];
          unpack8(packed, z);
          float n2 = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) n2 += z[i] * z[i];
          n2 = half_warp_sum(n2);
          const float nrm = sqrtf(n2) * (which == 0 ? p.q_norm_mult : 1.0f);
          // fold both rows of the warp access into the running per-head maximum kept by lane 0
          const float n_lo = __shfl_sync(0xffffffffu, nrm, 0), n_hi = __shfl_sync(0xffffffffu, nrm, 16);
          const int h_lo = __shfl_sync(0xffffffffu, hh[u], 0), h_hi = __shfl_sync(0xffffffffu, hh[u], 16);
          const bool in_hi = __shfl_sync(0xffffffffu, static_cast<int>(rid < rows), 16) != 0;
          const bool in_lo = __shfl_sync(0xffffffffu, static_cast<int>(rid < rows), 0) != 0;
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int h = e ? h_hi : h_lo;
            const float n = e ? n_hi : n_lo;
            if (!(e ? in_hi : in_lo)) continue;
            if (h != best_h) {
              if (best_h >= 0 && lane == 0) atomicMax(reinterpret_cast<int*>(p.norms + which * p.H + best_h), __float_as_int(best));
              best_h = h;
              best = 0.f;
            }
            best = fmaxf(best, n);
          }
        }
      }
      if (rid < rows) reinterpret_cast<uint4*>(p.out[which] + rid * kD)[hl] = packed;
    }
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
  const int64_t rows = static_cast<int64_t>(pp->B) * pp->H * pp->S;
  const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((rows + 31) / 32, 148 * 16));
  qk_prepass_kernel<<<dim3(blocks, kp.n_tensors), 256, 0, s>>>(kp);
  if (!launch_ok("qk_prepass_kernel launch")) return DTB_ERR_LAUNCH;
  if (pp->mk_out != nullptr) {
    prepass_bound_kernel<<<(pp->H + 127) / 128, 128, 0, s>>>(pp->norms, pp->H, pp->gate > 0.f ? pp->gate : 213.0f,
                                                             pp->mk_out);
    if (!launch_ok("prepass_bound_kernel launch")) return DTB_ERR_LAUNCH;
  }
  return DTB_OK;
}
