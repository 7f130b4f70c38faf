// k-smoothing: subtract from every key row the mean key of its (batch, head) over the valid rows, and zero the
// padded rows.  Softmax is invariant to it, and it makes every query row's mean logit exactly zero, hence its
// largest logit non-negative, which is what lets the bounded-logit softmax use the wide gate.
//
// Two kernels, both HBM-bound (one read of K each, the second also one write):
//   k_colsum_kernel  per (chunk of rows, head, batch): f32 column sums over the valid rows -> partial[chunk]
//   k_smooth_kernel  sums the partials in a fixed order (the result does not depend on scheduling), rounds the
//                    mean to bf16 as the reference does, writes bf16(k - mean) or zeros, and collects the
//                    largest output row norm per head for the bounded-logit operand.
// Sixteen lanes own a 256-byte row (8 elements each); a block of 256 threads takes 16 rows per step.
#include <algorithm>

#include "host_common.h"
#include "ptx.cuh"

namespace dtb {
namespace {

constexpr int kD = 128;
constexpr int kMaxChunks = DTB_SMOOTH_K_CHUNKS;

struct SmoothParams {
  const __nv_bfloat16* k;
  int64_t sb, sh, ss;
  __nv_bfloat16* out;
  int64_t ob, oh, os;
  const int32_t* kv_len;
  float* partial;      // [chunks, B, H, 128]
  float* norm_max;     // [H] or null
  int B, H, S, chunks, rows_per_chunk;
};

__device__ __forceinline__ void unpack8(const uint4& raw, float (&x)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    x[2 * i] = f.x;
    x[2 * i + 1] = f.y;
  }
}

__global__ void __launch_bounds__(256) k_colsum_kernel(const __grid_constant__ SmoothParams p) {
  __shared__ float red[16][kD];
  const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hl = threadIdx.x & 15;       // lane within the row
  const int rg = threadIdx.x >> 4;       // row group 0..15
  const int n_valid = p.kv_len != nullptr ? min(max(p.kv_len[b], 0), p.S) : p.S;
  const int r0 = chunk * p.rows_per_chunk;
  const int r1 = min(r0 + p.rows_per_chunk, n_valid);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const __nv_bfloat16* base = p.k + b * p.sb + h * p.sh;
  // four rows in flight per thread: the kernel lives on memory-level parallelism
  int r = r0 + rg;
  for (; r + 48 < r1; r += 64) {
    uint4 raw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) raw[u] = reinterpret_cast<const uint4*>(base + (r + 16 * u) * p.ss)[hl];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float x[8];
      unpack8(raw[u], x);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += x[i];
    }
  }
  for (; r < r1; r += 16) {
    float x[8];
    unpack8(reinterpret_cast<const uint4*>(base + r * p.ss)[hl], x);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += x[i];
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[rg][hl * 8 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < kD) {
    float s = 0.f;
#pragma unroll
    for (int g = 0; g < 16; ++g) s += red[g][threadIdx.x];
    p.partial[((static_cast<int64_t>(chunk) * p.B + b) * p.H + h) * kD + threadIdx.x] = s;
  }
}

__global__ void __launch_bounds__(256) k_smooth_kernel(const __grid_constant__ SmoothParams p) {
  __shared__ float mean_s[kD];
  __shared__ int max_s;
  const int chunk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hl = threadIdx.x & 15;
  const int rg = threadIdx.x >> 4;
  const int n_valid = p.kv_len != nullptr ? min(max(p.kv_len[b], 0), p.S) : p.S;
  if (threadIdx.x == 0) max_s = 0;
  if (threadIdx.x < kD) {
    float s = 0.f;
    for (int c = 0; c < p.chunks; ++c) s += p.partial[((static_cast<int64_t>(c) * p.B + b) * p.H + h) * kD + threadIdx.x];
    // the mean is rounded to the keys' dtype before the subtraction, as the reference does
    mean_s[threadIdx.x] = n_valid > 0 ? __bfloat162float(__float2bfloat16_rn(s / static_cast<float>(n_valid))) : 0.f;
  }
  __syncthreads();
  float mean[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) mean[i] = mean_s[hl * 8 + i];
  const int r0 = chunk * p.rows_per_chunk;
  const int r1 = min(r0 + p.rows_per_chunk, p.S);
  const __nv_bfloat16* src = p.k + b * p.sb + h * p.sh;
  __nv_bfloat16* dst = p.out + b * p.ob + h * p.oh;
  float best = 0.f;
  // the sixteen lanes of a row run the same number of steps; the other half of the warp may run one fewer,
  // so the row reduction names only its own half
  const uint32_t half_mask = 0xffffu << (threadIdx.x & 16);
  // two rows per step, both loads issued before either row is worked on
  auto finish_row = [&](int r, const uint4& raw, bool live) {
    uint4 packed = make_uint4(0u, 0u, 0u, 0u);
    float n2 = 0.f;
    if (live) {
      float x[8];
      unpack8(raw, x);
      uint32_t y[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) y[i] = pack_bf16x2(x[2 * i] - mean[2 * i], x[2 * i + 1] - mean[2 * i + 1]);
      packed = make_uint4(y[0], y[1], y[2], y[3]);
      float z[8];
      unpack8(packed, z);
#pragma unroll
      for (int i = 0; i < 8; ++i) n2 += z[i] * z[i];
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) n2 += __shfl_xor_sync(half_mask, n2, o);
    best = fmaxf(best, n2);
    reinterpret_cast<uint4*>(dst + r * p.os)[hl] = packed;
  };
  for (int r = r0 + rg; r < r1; r += 32) {
    const int rb = r + 16;
    const bool has_b = rb < r1;                      // the same for the sixteen lanes of a row
    const bool live_a = r < n_valid, live_b = has_b && rb < n_valid;
    uint4 raw_a = make_uint4(0u, 0u, 0u, 0u), raw_b = raw_a;
    if (live_a) raw_a = reinterpret_cast<const uint4*>(src + r * p.ss)[hl];
    if (live_b) raw_b = reinterpret_cast<const uint4*>(src + rb * p.ss)[hl];
    finish_row(r, raw_a, live_a);
    if (has_b) finish_row(rb, raw_b, live_b);
  }
  if (p.norm_max != nullptr) {
    if (hl == 0 && best > 0.f) atomicMax(&max_s, __float_as_int(sqrtf(best)));
    __syncthreads();
    if (threadIdx.x == 0 && max_s != 0) atomicMax(reinterpret_cast<int*>(p.norm_max + h), max_s);
  }
}

__global__ void mk_from_norms_kernel(const float* __restrict__ qn, const float* __restrict__ kn, int Hq, int Hkv,
                                     float gate, float* __restrict__ mk) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= Hq) return;
  const float bound = qn[h] * kn[h / (Hq / Hkv)];
  mk[h] = ceilf(bound);
  mk[Hq + h] = (bound <= gate) ? 1.0f : 0.0f;
}

}  // namespace
}  // namespace dtb

extern "C" size_t dtb_smooth_k_scratch_bytes(int32_t B, int32_t H) {
  if (B <= 0 || H <= 0) return 0;
  return static_cast<size_t>(dtb::kMaxChunks) * B * H * dtb::kD * sizeof(float);
}

extern "C" int dtb_smooth_k(const dtb_smooth_k_params* sp, void* stream) {
  using namespace dtb;
  if (sp == nullptr || sp->k == nullptr || sp->out == nullptr || sp->scratch == nullptr) return DTB_ERR_NULL;
  if (sp->D != kD || sp->B <= 0 || sp->H <= 0 || sp->S <= 0 || sp->H > 65535 || sp->B > 65535) return DTB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(sp->k) & 15u) || (reinterpret_cast<uintptr_t>(sp->out) & 15u) ||
      (reinterpret_cast<uintptr_t>(sp->scratch) & 3u))
    return DTB_ERR_ALIGN;
  const int64_t strides[6] = {sp->k_stride_b, sp->k_stride_h, sp->k_stride_s, sp->out_stride_b, sp->out_stride_h,
                              sp->out_stride_s};
  for (int64_t s : strides)
    if (s & 7) return DTB_ERR_ALIGN;
  if (sp->k_stride_s <= 0 || sp->out_stride_s <= 0) return DTB_ERR_SHAPE;
  if (sp->scratch_bytes < dtb_smooth_k_scratch_bytes(sp->B, sp->H)) return DTB_ERR_WORKSPACE;
  SmoothParams kp;
  kp.k = static_cast<const __nv_bfloat16*>(sp->k);
  kp.sb = sp->k_stride_b; kp.sh = sp->k_stride_h; kp.ss = sp->k_stride_s;
  kp.out = static_cast<__nv_bfloat16*>(sp->out);
  kp.ob = sp->out_stride_b; kp.oh = sp->out_stride_h; kp.os = sp->out_stride_s;
  kp.kv_len = sp->kv_len;
  kp.partial = static_cast<float*>(sp->scratch);
  kp.norm_max = sp->k_norm_max;
  kp.B = sp->B; kp.H = sp->H; kp.S = sp->S;
  kp.chunks = std::max(1, std::min(kMaxChunks, (sp->S + 255) / 256));
  kp.rows_per_chunk = (sp->S + kp.chunks - 1) / kp.chunks;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (sp->k_norm_max != nullptr &&
      !cuda_ok(cudaMemsetAsync(sp->k_norm_max, 0, sizeof(float) * sp->H, s), "cudaMemsetAsync(k_norm_max)"))
    return DTB_ERR_LAUNCH;
  const dim3 grid(kp.chunks, sp->H, sp->B);
  k_colsum_kernel<<<grid, 256, 0, s>>>(kp);
  if (!launch_ok("k_colsum_kernel launch")) return DTB_ERR_LAUNCH;
  k_smooth_kernel<<<grid, 256, 0, s>>>(kp);
  return launch_ok("k_smooth_kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}

extern "C" int dtb_fixed_m_from_norms(const float* q_norms, const float* k_norms, int32_t Hq, int32_t Hkv, float gate,
                                      float* mk_out, void* stream) {
  using namespace dtb;
  if (q_norms == nullptr || k_norms == nullptr || mk_out == nullptr) return DTB_ERR_NULL;
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0) return DTB_ERR_SHAPE;
  mk_from_norms_kernel<<<(Hq + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      q_norms, k_norms, Hq, Hkv, gate > 0.f ? gate : 213.0f, mk_out);
  return launch_ok("mk_from_norms_kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}
