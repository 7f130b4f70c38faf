// C-ABI entry points of the attention forward: argument checking, tensor-map
// encoding, variant selection (plain / split-KV / residual) and the small helper
// kernels around the main one (partial-state combine, bounded-logit operand).
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <mutex>

#include <cuda_fp8.h>

#include "attn_kernel.cuh"
#include "host_common.h"

namespace dtb {
namespace {

constexpr float kLog2e = 1.44269504f;
constexpr int kNumSms = 148;

// ---------------------------------------------------------------------------
// Merge `num` partial states per row and write the normalised bf16 output.
// One warp per query row; lane i owns output columns 4i..4i+3.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) combine_kernel(const float* __restrict__ acc_o, const float* __restrict__ acc_m,
                                                      const float* __restrict__ acc_l, int num, int B, int Hq, int Sq,
                                                      __nv_bfloat16* __restrict__ o, int64_t osb, int64_t osh,
                                                      int64_t oss, const int32_t* __restrict__ kv_len, int q_offset,
                                                      int zero_padded_rows) {
  const int64_t rows = static_cast<int64_t>(B) * Hq * Sq;
  const int64_t rid = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (rid >= rows) return;
  const int lane = threadIdx.x & 31;
  const int s = static_cast<int>(rid % Sq);
  const int h = static_cast<int>((rid / Sq) % Hq);
  const int b = static_cast<int>(rid / (static_cast<int64_t>(Sq) * Hq));
  float m_max = -INFINITY;
  for (int i = 0; i < num; ++i) {
    const float l = acc_l[i * rows + rid];
    const float m = acc_m[i * rows + rid];
    if (l > 0.f) m_max = fmaxf(m_max, m);
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float l_tot = 0.f;
  for (int i = 0; i < num; ++i) {
    const float l = acc_l[i * rows + rid];
    if (!(l > 0.f)) continue;
    const float w = exp2f(acc_m[i * rows + rid] - m_max);
    l_tot += l * w;
    const float4 v = reinterpret_cast<const float4*>(acc_o + (i * rows + rid) * kHeadDim)[lane];
    acc.x += v.x * w;
    acc.y += v.y * w;
    acc.z += v.z * w;
    acc.w += v.w * w;
  }
  const bool padded = zero_padded_rows && kv_len != nullptr && (q_offset + s >= kv_len[b]);
  const float inv = (l_tot > 0.f && !padded) ? 1.0f / l_tot : 0.f;
  uint2 packed;
  packed.x = pack_bf16x2(acc.x * inv, acc.y * inv);
  packed.y = pack_bf16x2(acc.z * inv, acc.w * inv);
  reinterpret_cast<uint2*>(o + b * osb + h * osh + s * oss)[lane] = packed;
}

// ---------------------------------------------------------------------------
// Merge of a balanced launch: the units of the last wave were swept in pieces, whose (o, m, l) lie in
// consecutive scratch slots per unit (256 rows each).  One warp per query row; lane i owns columns 4i..4i+3.
// ---------------------------------------------------------------------------
struct PeerOut {                     // sequence-sharded output of a head-parallel call (shard_rows == 0: none)
  __nv_bfloat16* o_peer[8];
  int shard_rows, total_heads, head_offset;
};

struct PieceMerge {
  int first_unit;                    // unit index of tail unit 0
  int n_units;                       // tail units
  int q_blocks;
  uint16_t slot_base[148];           // first slot of tail unit x
  uint8_t slot_count[148];           // its number of slots (0: the unit was swept whole, nothing to merge)
};

__global__ void __launch_bounds__(256) merge_pieces_kernel(const __grid_constant__ PieceMerge pm,
                                                           const __grid_constant__ PeerOut po,
                                                           const float* __restrict__ acc_o, const float* __restrict__ acc_m,
                                                           const float* __restrict__ acc_l, int Hq, int Sq,
                                                           __nv_bfloat16* __restrict__ o, int64_t osb, int64_t osh,
                                                           int64_t oss, const int32_t* __restrict__ kv_len,
                                                           int zero_padded_rows) {
  constexpr int kRows = kQTiles * kBlockM;
  const int x = blockIdx.x / (kRows / 8);
  const int r = (blockIdx.x % (kRows / 8)) * 8 + (threadIdx.x >> 5);
  const int count = pm.slot_count[x];
  if (count == 0) return;
  const int lane = threadIdx.x & 31;
  // everything above is independent of the sweep kernel; its results are needed from here on
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int unit = pm.first_unit + x;
  const int qb = unit % pm.q_blocks;
  const int bh = unit / pm.q_blocks;
  const int h = bh % Hq, b = bh / Hq;
  const int s = qb * kRows + r;
  if (s >= Sq) return;
  const int64_t row0 = static_cast<int64_t>(pm.slot_base[x]) * kRows + r;
  // Pieces are taken four at a time with all their loads issued before any is used: the kernel is bound by
  // the latency of these loads, not by their volume.
  float m_max = -INFINITY;
  for (int i0 = 0; i0 < count; i0 += 4) {
    float l4[4], m4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t rr = row0 + static_cast<int64_t>(min(i0 + u, count - 1)) * kRows;
      l4[u] = acc_l[rr];
      m4[u] = acc_m[rr];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i0 + u < count && l4[u] > 0.f) m_max = fmaxf(m_max, m4[u]);
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float l_tot = 0.f;
  for (int i0 = 0; i0 < count; i0 += 4) {
    float l4[4], m4[4];
    float4 v4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t rr = row0 + static_cast<int64_t>(min(i0 + u, count - 1)) * kRows;
      l4[u] = acc_l[rr];
      m4[u] = acc_m[rr];
      v4[u] = reinterpret_cast<const float4*>(acc_o + rr * kHeadDim)[lane];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (i0 + u < count && l4[u] > 0.f) {     // a piece with no valid key wrote no o: never touch it
        const float w = exp2f(m4[u] - m_max);
        l_tot += l4[u] * w;
        acc.x += v4[u].x * w;
        acc.y += v4[u].y * w;
        acc.z += v4[u].z * w;
        acc.w += v4[u].w * w;
      }
    }
  }
  const bool padded = zero_padded_rows && kv_len != nullptr && (s >= kv_len[b]);
  const float inv = (l_tot > 0.f && !padded) ? 1.0f / l_tot : 0.f;
  uint2 packed;
  packed.x = pack_bf16x2(acc.x * inv, acc.y * inv);
  packed.y = pack_bf16x2(acc.z * inv, acc.w * inv);
  __nv_bfloat16* dst = o + b * osb + h * osh + s * oss;
  if (po.shard_rows > 0) {
    const int dest = s / po.shard_rows;
    dst = po.o_peer[dest] + ((static_cast<int64_t>(b) * po.total_heads + po.head_offset + h) * po.shard_rows +
                             (s - dest * po.shard_rows)) * kHeadDim;
  }
  reinterpret_cast<uint2*>(dst)[lane] = packed;
}

// ---------------------------------------------------------------------------
// Max L2 row norm per head of a bf16 [B,H,S,128] tensor (one warp per row),
// folded into norms[h] with an integer atomic max (norms are non-negative).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) row_norm_max_kernel(const __nv_bfloat16* __restrict__ x, int B, int H, int S,
                                                           int64_t sb, int64_t sh, int64_t ss, float mult,
                                                           float* __restrict__ norms) {
  const int64_t rows = static_cast<int64_t>(B) * H * S;
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * 8;
  float best = 0.f;
  int best_h = -1;
  for (int64_t rid = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); rid < rows; rid += warps_total) {
    // rows are visited head-major so one warp mostly stays inside one head
    const int s = static_cast<int>(rid % S);
    const int b = static_cast<int>((rid / S) % B);
    const int h = static_cast<int>(rid / (static_cast<int64_t>(S) * B));
    if (h != best_h) {
      if (best_h >= 0 && lane == 0) atomicMax(reinterpret_cast<int*>(norms + best_h), __float_as_int(best));
      best_h = h;
      best = 0.f;
    }
    const uint2 raw = reinterpret_cast<const uint2*>(x + b * sb + h * sh + s * ss)[lane];
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    float ss2 = a.x * a.x + a.y * a.y + c.x * c.x + c.y * c.y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss2 += __shfl_xor_sync(0xffffffffu, ss2, o);
    best = fmaxf(best, sqrtf(ss2) * mult);
  }
  if (best_h >= 0 && lane == 0) atomicMax(reinterpret_cast<int*>(norms + best_h), __float_as_int(best));
}

__global__ void fixed_m_finish_kernel(const float* __restrict__ norms, int Hq, int Hkv, float gate,
                                      float* __restrict__ mk) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= Hq) return;
  const float bound = norms[h] * norms[Hq + h / (Hq / Hkv)];
  mk[h] = ceilf(bound);
  mk[Hq + h] = (bound <= gate) ? 1.0f : 0.0f;
}

// ---------------------------------------------------------------------------
// Sequence shards -> head shards without an intermediate copy: rank `rank` holds x[B, H, Sl, D] (all
// heads of its sequence shard) and writes head group r of it straight into rank r's buffer
// y_r[B, H/P, P*Sl, D] at rows [rank*Sl, (rank+1)*Sl), 16 bytes per thread, 256-byte rows coalesced.
// Destinations may be peer memory (plain stores over NVLink).  grid.y selects one of up to 3 tensors.
// ---------------------------------------------------------------------------
struct ScatterHeadsParams {
  const __nv_bfloat16* src[3];
  int64_t sb[3], sh[3], ss[3];
  __nv_bfloat16* dst[3][8];
  int B, H, Sl, P, rank;
};

__global__ void __launch_bounds__(256) scatter_heads_kernel(const __grid_constant__ ScatterHeadsParams sp) {
  const int which = blockIdx.y;
  const int Hl = sp.H / sp.P;
  const int64_t chunks = static_cast<int64_t>(sp.B) * sp.H * sp.Sl * 16;   // 16-byte chunks
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < chunks;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx & 15);
    const int64_t rowid = idx >> 4;
    const int sl = static_cast<int>(rowid % sp.Sl);
    const int h = static_cast<int>((rowid / sp.Sl) % sp.H);
    const int b = static_cast<int>(rowid / (static_cast<int64_t>(sp.Sl) * sp.H));
    const uint4 v = reinterpret_cast<const uint4*>(sp.src[which] + b * sp.sb[which] + h * sp.sh[which] + sl * sp.ss[which])[c];
    const int r = h / Hl;
    __nv_bfloat16* drow = sp.dst[which][r] +
                          ((static_cast<int64_t>(b) * Hl + (h - r * Hl)) * (static_cast<int64_t>(sp.P) * sp.Sl) +
                           static_cast<int64_t>(sp.rank) * sp.Sl + sl) * kHeadDim;
    reinterpret_cast<uint4*>(drow)[c] = v;
  }
}

// ---------------------------------------------------------------------------
int check_params(const dtb_attn_params* p, bool need_o) {
  if (p == nullptr || p->q == nullptr || p->k == nullptr || p->v == nullptr) return DTB_ERR_NULL;
  if (need_o && p->o == nullptr) return DTB_ERR_NULL;
  if (p->D != kHeadDim) return DTB_ERR_SHAPE;
  if (p->B <= 0 || p->Hq <= 0 || p->Hkv <= 0 || p->Sq <= 0 || p->Skv <= 0) return DTB_ERR_SHAPE;
  if (p->Hq % p->Hkv != 0) return DTB_ERR_SHAPE;
  if (p->Hq > 65535 || static_cast<int64_t>(p->B) * 64 > 65535) return DTB_ERR_SHAPE;
  // an axis of extent > 1 must have a positive stride (no broadcast or reversed views)
  if (p->q_stride_s <= 0 || p->k_stride_s <= 0 || p->v_stride_s <= 0) return DTB_ERR_SHAPE;
  if (p->Hq > 1 && p->q_stride_h <= 0) return DTB_ERR_SHAPE;
  if (p->Hkv > 1 && (p->k_stride_h <= 0 || p->v_stride_h <= 0)) return DTB_ERR_SHAPE;
  if (p->B > 1 && (p->q_stride_b <= 0 || p->k_stride_b <= 0 || p->v_stride_b <= 0)) return DTB_ERR_SHAPE;
  if (need_o) {
    if (reinterpret_cast<uintptr_t>(p->o) & 15u) return DTB_ERR_ALIGN;
    if ((p->o_stride_s * 2) & 15 || (p->o_stride_h * 2) & 15 || (p->o_stride_b * 2) & 15) return DTB_ERR_ALIGN;
  }
  if ((p->flags & DTB_FLAG_BOUNDED_LOGITS) && p->mk == nullptr) return DTB_ERR_NULL;
  return DTB_OK;
}

int q_blocks(const dtb_attn_params* p) { return (p->Sq + kQTiles * kBlockM - 1) / (kQTiles * kBlockM); }

// Split-KV factor.  Splitting pays when the (batch, head, query-block) grid leaves
// most SMs idle and each CTA would otherwise sweep many key tiles alone.
int resolve_splits(const dtb_attn_params* p) {
  if (p->num_splits == 1 || (p->flags & DTB_FLAG_QK_FP8)) return 1;
  const int kv_tiles = (p->Skv + kBlockN - 1) / kBlockN;
  int n = p->num_splits;
  if (n <= 0) {
    const int64_t ctas = static_cast<int64_t>(q_blocks(p)) * p->Hq * p->B;
    if (ctas * 2 > kNumSms || kv_tiles < 8) return 1;
    n = static_cast<int>(kNumSms / ctas);
    n = std::min(n, kv_tiles / 4);
  }
  n = std::min(n, std::min(kv_tiles, 64));
  return std::max(n, 1);
}

int current_sm_count() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) == cudaSuccess &&
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0)
    return std::min(sms, 148);
  (void)cudaGetLastError();
  return kNumSms;   // no device to ask (sizing queries on a machine without one): a B200's count
}

// ---------------------------------------------------------------------------
// Balanced launch (the role of the reference's per-shape tile resolution, diffusers_tpu/kernels/block_sizes.py:442-577,
// resolved from the static shape alone as in diffusers_tpu/kernels/mesh_attention.py:199-216): with one CTA per
// (batch, head, query block) unit the last wave of a launch leaves SMs idle - a whole sweep long when the units
// do not fill it.  When that costs a tenth of the sweep or more, the key tiles of the last wave's units are
// cut into `sms` runs of equal length; a run that crosses a unit boundary becomes two pieces.  Pieces of one unit
// get consecutive scratch slots and are merged by merge_pieces_kernel.
// ---------------------------------------------------------------------------
constexpr int kMinPieceTiles = 4;      // no run shorter than this many key tiles
// What the balanced form costs an SM beyond its run of key tiles, in key-tile times: a second pipeline fill and
// drain (a run usually spans two units), the state written instead of the output, and the merge kernel.
#ifndef DTB_PIECE_OVERHEAD_TILES
#define DTB_PIECE_OVERHEAD_TILES 13
#endif
constexpr int kPieceOverheadTiles = DTB_PIECE_OVERHEAD_TILES;

struct BalancedPlan {
  bool use = false;
  int slots = 0;
  PieceTable table;
  PieceMerge merge;
};

void plan_balanced(const dtb_attn_params* p, int sms, BalancedPlan* plan) {
  plan->use = false;
  plan->slots = 0;
  const int qb = q_blocks(p);
  const long long units = static_cast<long long>(qb) * p->Hq * p->B;
  const int n = (p->Skv + kBlockN - 1) / kBlockN;
  if (units > 0x7fffffffLL || n > 65535) return;
  const int tail = static_cast<int>(units % sms);
  if (tail == 0) return;
  const long long tiles = static_cast<long long>(tail) * n;
  const int runs = static_cast<int>(std::min<long long>(sms, tiles / kMinPieceTiles));
  if (runs <= tail) return;
  const long long run_len = (tiles + runs - 1) / runs;
  if (run_len + kPieceOverheadTiles > n) return;   // the plain launch is as fast or faster
  struct Piece { int x, tb, te; };
  Piece pieces[kMaxPieces];
  int np = 0;
  for (int i = 0; i < runs; ++i) {
    long long s0 = tiles * i / runs, s1 = tiles * (i + 1) / runs;
    while (s0 < s1) {
      const int x = static_cast<int>(s0 / n);
      const long long end = std::min<long long>(s1, static_cast<long long>(x + 1) * n);
      if (np >= kMaxPieces) return;
      pieces[np++] = {x, static_cast<int>(s0 - static_cast<long long>(x) * n), static_cast<int>(end - static_cast<long long>(x) * n)};
      s0 = end;
    }
  }
  // slots: consecutive per unit, in the order of the key ranges (pieces are generated in that order)
  PieceMerge& mg = plan->merge;
  mg.first_unit = static_cast<int>(units - tail);
  mg.n_units = tail;
  mg.q_blocks = qb;
  for (int x = 0; x < 148; ++x) { mg.slot_base[x] = 0; mg.slot_count[x] = 0; }
  int slot_of[kMaxPieces];
  int slots = 0;
  for (int i = 0; i < np; ++i) {
    const bool whole = pieces[i].tb == 0 && pieces[i].te == n;
    if (whole) { slot_of[i] = -1; continue; }
    if (mg.slot_count[pieces[i].x] == 0) mg.slot_base[pieces[i].x] = static_cast<uint16_t>(slots);
    if (mg.slot_count[pieces[i].x] == 255) return;
    mg.slot_count[pieces[i].x]++;
    slot_of[i] = slots++;
  }
  // longest pieces first
  int order[kMaxPieces];
  for (int i = 0; i < np; ++i) order[i] = i;
  std::stable_sort(order, order + np, [&](int a, int b) {
    return pieces[a].te - pieces[a].tb > pieces[b].te - pieces[b].tb;
  });
  PieceTable& tb = plan->table;
  tb.whole_units = mg.first_unit;
  tb.n_pieces = np;
  tb.q_blocks = qb;
  for (int k = 0; k < np; ++k) {
    const Piece& pc = pieces[order[k]];
    tb.unit[k] = mg.first_unit + pc.x;
    tb.tile_begin[k] = static_cast<uint16_t>(pc.tb);
    tb.tile_end[k] = static_cast<uint16_t>(pc.te);
    tb.slot[k] = static_cast<int16_t>(slot_of[order[k]]);
  }
  for (int k = np; k < kMaxPieces; ++k) { tb.unit[k] = 0; tb.tile_begin[k] = tb.tile_end[k] = 0; tb.slot[k] = -1; }
  plan->slots = slots;
  plan->use = slots > 0;
}

size_t balanced_workspace_bytes(int slots) {
  return static_cast<size_t>(slots) * (kQTiles * kBlockM) * (kHeadDim + 2) * sizeof(float);
}

size_t split_workspace_bytes(const dtb_attn_params* p, int splits) {
  const size_t rows = static_cast<size_t>(splits) * p->B * p->Hq * p->Sq;
  return rows * (kHeadDim + 2) * sizeof(float);
}

// The opt-in shared-memory size is a per-device function attribute: set it the first
// time each device is used (an immutable cache; nothing else in the library is global).
std::atomic<bool> g_attrs_set[64];

cudaError_t ensure_kernel_attrs() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && g_attrs_set[dev].load(std::memory_order_acquire)) return cudaSuccess;
  e = cudaFuncSetAttribute(attn_fwd_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kSmemBytes));
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(attn_fwd_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kSmemBytes));
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(attn_fwd_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kSmemBytes));
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(attn_fwd_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kSmemBytes));
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(attn_fwd_pieces_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kSmemBytes));
  if (e != cudaSuccess) return e;
  // The register hand-over inside the kernel (setmaxnreg) is sized for kLaunchRegs registers per thread at
  // launch; with any other count a warpgroup could wait for registers that never come.  Refuse to launch then.
  const void* variants[5] = {reinterpret_cast<const void*>(attn_fwd_kernel<false, false>),
                             reinterpret_cast<const void*>(attn_fwd_kernel<true, false>),
                             reinterpret_cast<const void*>(attn_fwd_kernel<false, true>),
                             reinterpret_cast<const void*>(attn_fwd_kernel<true, true>),
                             reinterpret_cast<const void*>(attn_fwd_pieces_kernel)};
  for (const void* fn : variants) {
    cudaFuncAttributes fa;
    e = cudaFuncGetAttributes(&fa, fn);
    if (e != cudaSuccess) return e;
    if (fa.numRegs != kLaunchRegs) return cudaErrorInvalidConfiguration;
  }
  if (dev >= 0 && dev < 64) g_attrs_set[dev].store(true, std::memory_order_release);
  return cudaSuccess;
}

int fill_kernel_params(const dtb_attn_params* p, AttnKernelParams* kp) {
  const bool fp8 = (p->flags & DTB_FLAG_QK_FP8) != 0;
  int st = fp8 ? make_tmap_bhsd_u8(&kp->tmap_q, p->q, p->B, p->Hq, p->Sq, p->q_stride_b, p->q_stride_h, p->q_stride_s,
                                   kBlockM)
               : make_tmap_bhsd(&kp->tmap_q, p->q, p->B, p->Hq, p->Sq, p->q_stride_b, p->q_stride_h, p->q_stride_s,
                                kBlockM);
  if (st != DTB_OK) return st;
  st = fp8 ? make_tmap_bhsd_u8(&kp->tmap_k, p->k, p->B, p->Hkv, p->Skv, p->k_stride_b, p->k_stride_h, p->k_stride_s,
                               kBlockN)
           : make_tmap_bhsd(&kp->tmap_k, p->k, p->B, p->Hkv, p->Skv, p->k_stride_b, p->k_stride_h, p->k_stride_s,
                            kBlockN);
  if (st != DTB_OK) return st;
  st = make_tmap_bhsd(&kp->tmap_v, p->v, p->B, p->Hkv, p->Skv, p->v_stride_b, p->v_stride_h, p->v_stride_s,
                      kBlockN);
  if (st != DTB_OK) return st;
  kp->o = static_cast<__nv_bfloat16*>(p->o);
  kp->o_stride_b = p->o_stride_b;
  kp->o_stride_h = p->o_stride_h;
  kp->o_stride_s = p->o_stride_s;
  kp->acc_o = kp->acc_m = kp->acc_l = nullptr;
  kp->kv_len = p->kv_len;
  kp->mk = (p->flags & DTB_FLAG_BOUNDED_LOGITS) ? p->mk : nullptr;
  kp->status = p->status;
  kp->B = p->B;
  kp->Hq = p->Hq;
  kp->Hkv = p->Hkv;
  kp->Sq = p->Sq;
  kp->Skv = p->Skv;
  kp->kv_offset = 0;
  kp->q_offset = 0;
  kp->num_splits = 1;
  kp->acc_init = 1;
  kp->zero_padded_rows = (p->flags & DTB_FLAG_ZERO_PADDED_ROWS) ? 1 : 0;
  const float scale = p->scale > 0.f ? p->scale : 1.0f / sqrtf(static_cast<float>(p->D));
  kp->scale_log2 = scale * kLog2e;
  for (int i = 0; i < 8; ++i) kp->o_peer[i] = nullptr;
  kp->o_shard_rows = 0;
  kp->o_total_heads = 0;
  kp->o_head_offset = 0;
  kp->kv_table = nullptr;
  kp->kv_count = nullptr;
  kp->head_class = nullptr;
  kp->table_qblocks = 0;
  kp->table_width = 0;
  return DTB_OK;
}

// Sweep with the last wave in pieces, then the merge (see plan_balanced).  `workspace` holds
// balanced_workspace_bytes(plan.slots) bytes.
int launch_balanced(const dtb_attn_params* p, AttnKernelParams kp, const BalancedPlan& plan, void* workspace,
                    cudaStream_t s) {
  const size_t rows = static_cast<size_t>(plan.slots) * (kQTiles * kBlockM);
  kp.acc_o = static_cast<float*>(workspace);
  kp.acc_m = kp.acc_o + rows * kHeadDim;
  kp.acc_l = kp.acc_m + rows;
  kp.acc_init = 1;
  attn_fwd_pieces_kernel<<<dim3(plan.table.whole_units + plan.table.n_pieces), dim3(kNumThreads), kSmemBytes, s>>>(
      kp, plan.table);
  if (!launch_ok("attn_fwd_pieces_kernel launch")) return DTB_ERR_LAUNCH;
  PeerOut po;
  for (int i = 0; i < 8; ++i) po.o_peer[i] = kp.o_peer[i];
  po.shard_rows = kp.o_shard_rows;
  po.total_heads = kp.o_total_heads;
  po.head_offset = kp.o_head_offset;
  // The merge is launched as a programmatic dependent of the sweep: its blocks are set up while the sweep
  // drains and wait (griddepcontrol.wait in the kernel) until all of the sweep's writes are visible.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(plan.merge.n_units * (kQTiles * kBlockM / 8));
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const float* c_o = kp.acc_o;
  const float* c_m = kp.acc_m;
  const float* c_l = kp.acc_l;
  if (!cuda_ok(cudaLaunchKernelEx(&cfg, merge_pieces_kernel, plan.merge, po, c_o, c_m, c_l, static_cast<int>(p->Hq),
                                  static_cast<int>(p->Sq), kp.o, kp.o_stride_b, kp.o_stride_h, kp.o_stride_s,
                                  p->kv_len, kp.zero_padded_rows),
               "merge_pieces_kernel launch"))
    return DTB_ERR_LAUNCH;
  return DTB_OK;
}

}  // namespace
}  // namespace dtb

using namespace dtb;

extern "C" int dtb_attn_supported(const dtb_attn_params* p, int* why) {
  int st = check_params(p, true);
  if (st == DTB_OK && !device_is_sm100()) st = DTB_ERR_ARCH;
  if (why != nullptr) *why = st;
  return st == DTB_OK ? 1 : 0;
}

extern "C" size_t dtb_attn_workspace_bytes(const dtb_attn_params* p) {
  if (check_params(p, false) != DTB_OK) return 0;
  if (p->num_splits == 0 && !(p->flags & DTB_FLAG_QK_FP8)) {
    BalancedPlan plan;
    plan_balanced(p, current_sm_count(), &plan);
    return plan.use ? balanced_workspace_bytes(plan.slots) : 0;
  }
  const int splits = resolve_splits(p);
  return splits > 1 ? split_workspace_bytes(p, splits) : 0;
}

extern "C" int dtb_attn_launch_plan(const dtb_attn_params* p, int32_t sms, dtb_launch_plan* out) {
  static_assert(DTB_MAX_PIECES == kMaxPieces, "the public plan mirrors the kernel's piece table");
  int st = check_params(p, false);
  if (st != DTB_OK) return st;
  if (out == nullptr) return DTB_ERR_NULL;
  if (sms < 0 || sms > 148) return DTB_ERR_SHAPE;
  if (sms == 0) sms = current_sm_count();
  BalancedPlan plan;
  if (p->num_splits == 0 && !(p->flags & DTB_FLAG_QK_FP8)) plan_balanced(p, sms, &plan);
  const long long units = static_cast<long long>(q_blocks(p)) * p->Hq * p->B;
  out->units = static_cast<int32_t>(units);
  out->key_tiles = (p->Skv + kBlockN - 1) / kBlockN;
  out->tail_units = static_cast<int32_t>(units % sms);
  out->whole_units = plan.use ? plan.table.whole_units : static_cast<int32_t>(units);
  out->n_pieces = plan.use ? plan.table.n_pieces : 0;
  out->n_slots = plan.use ? plan.slots : 0;
  for (int i = 0; i < DTB_MAX_PIECES; ++i) {
    const bool live = plan.use && i < plan.table.n_pieces;
    out->unit[i] = live ? plan.table.unit[i] : 0;
    out->tile_begin[i] = live ? plan.table.tile_begin[i] : 0;
    out->tile_end[i] = live ? plan.table.tile_end[i] : 0;
    out->slot[i] = live ? plan.table.slot[i] : -1;
  }
  return DTB_OK;
}

extern "C" int dtb_attn_fwd(const dtb_attn_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  int st = check_params(p, true);
  if (st != DTB_OK) return st;
  if (!device_is_sm100()) return DTB_ERR_ARCH;
  if (!cuda_ok(ensure_kernel_attrs(), "attention kernel attributes (dynamic shared memory size; registers per thread as compiled)")) return DTB_ERR_LAUNCH;
  AttnKernelParams kp;
  st = fill_kernel_params(p, &kp);
  if (st != DTB_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  if (p->num_splits == 0 && !(p->flags & DTB_FLAG_QK_FP8)) {
    // automatic: one CTA per unit, the last wave balanced over the SMs when that pays and the caller's scratch
    // holds the pieces (a missing or smaller workspace is not an error: the plain launch runs instead)
    BalancedPlan plan;
    plan_balanced(p, current_sm_count(), &plan);
    if (plan.use) {
      if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 15u)) return DTB_ERR_ALIGN;
      if (workspace == nullptr || workspace_bytes < balanced_workspace_bytes(plan.slots)) plan.use = false;
    }
    if (plan.use) return launch_balanced(p, kp, plan, workspace, s);
    attn_fwd_kernel<false, false><<<dim3(q_blocks(p), p->Hq, p->B), dim3(kNumThreads), kSmemBytes, s>>>(kp);
    return launch_ok("kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
  }

  int splits = resolve_splits(p);
  if (splits > 1) {
    const size_t need = split_workspace_bytes(p, splits);
    if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 15u)) return DTB_ERR_ALIGN;
    if (workspace == nullptr || workspace_bytes < need) {
      if (p->num_splits > 1) return DTB_ERR_WORKSPACE;  // explicitly requested: refuse
      splits = 1;                                       // automatic: run unsplit
    }
  }
  const dim3 block(kNumThreads);
  if (p->flags & DTB_FLAG_QK_FP8) {
    // E4M3 q/k: one kernel variant, no split-KV
    if (p->num_splits > 1) return DTB_ERR_UNSUPPORTED;
    attn_fwd_kernel<false, true><<<dim3(q_blocks(p), p->Hq, p->B), block, kSmemBytes, s>>>(kp);
    return launch_ok("kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
  }
  if (splits == 1) {
    const dim3 grid(q_blocks(p), p->Hq, p->B);
    attn_fwd_kernel<false, false><<<grid, block, kSmemBytes, s>>>(kp);
    return launch_ok("kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
  }
  const size_t rows = static_cast<size_t>(splits) * p->B * p->Hq * p->Sq;
  kp.acc_o = static_cast<float*>(workspace);
  kp.acc_m = kp.acc_o + rows * kHeadDim;
  kp.acc_l = kp.acc_m + rows;
  kp.num_splits = splits;
  kp.acc_init = 1;
  const dim3 grid(q_blocks(p), p->Hq, p->B * splits);
  attn_fwd_kernel<true, false><<<grid, block, kSmemBytes, s>>>(kp);
  if (!launch_ok("attn_fwd_kernel launch")) return DTB_ERR_LAUNCH;
  const int64_t out_rows = static_cast<int64_t>(p->B) * p->Hq * p->Sq;
  combine_kernel<<<static_cast<unsigned>((out_rows + 7) / 8), 256, 0, s>>>(
      kp.acc_o, kp.acc_m, kp.acc_l, splits, p->B, p->Hq, p->Sq, kp.o, kp.o_stride_b, kp.o_stride_h, kp.o_stride_s,
      p->kv_len, 0, kp.zero_padded_rows);
  return launch_ok("kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}

extern "C" int dtb_attn_fwd_residual(const dtb_attn_params* p, const dtb_attn_residual* r, void* stream) {
  int st = check_params(p, false);
  if (st != DTB_OK) return st;
  if (r == nullptr || r->o_acc == nullptr || r->m == nullptr || r->l == nullptr) return DTB_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(r->o_acc) & 15u) return DTB_ERR_ALIGN;
  if (!device_is_sm100()) return DTB_ERR_ARCH;
  if (!cuda_ok(ensure_kernel_attrs(), "attention kernel attributes (dynamic shared memory size; registers per thread as compiled)")) return DTB_ERR_LAUNCH;
  AttnKernelParams kp;
  st = fill_kernel_params(p, &kp);
  if (st != DTB_OK) return st;
  kp.acc_o = r->o_acc;
  kp.acc_m = r->m;
  kp.acc_l = r->l;
  kp.kv_offset = r->kv_offset;
  kp.q_offset = r->q_offset;
  kp.acc_init = r->init ? 1 : 0;
  kp.zero_padded_rows = 0;  // padded rows are zeroed by dtb_attn_finalize
  const dim3 grid(q_blocks(p), p->Hq, p->B);
  if (p->flags & DTB_FLAG_QK_FP8)
    attn_fwd_kernel<true, true><<<grid, dim3(kNumThreads), kSmemBytes, static_cast<cudaStream_t>(stream)>>>(kp);
  else
    attn_fwd_kernel<true, false><<<grid, dim3(kNumThreads), kSmemBytes, static_cast<cudaStream_t>(stream)>>>(kp);
  return launch_ok("kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}

extern "C" int dtb_attn_finalize(const dtb_attn_params* p, const dtb_attn_residual* r, void* stream) {
  if (p == nullptr || p->o == nullptr || r == nullptr || r->o_acc == nullptr || r->m == nullptr || r->l == nullptr)
    return DTB_ERR_NULL;
  if (p->D != kHeadDim || p->B <= 0 || p->Hq <= 0 || p->Sq <= 0) return DTB_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(r->o_acc) & 15u) return DTB_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(p->o) & 7u) || (p->o_stride_s & 3) || (p->o_stride_h & 3) || (p->o_stride_b & 3))
    return DTB_ERR_ALIGN;
  const int64_t out_rows = static_cast<int64_t>(p->B) * p->Hq * p->Sq;
  combine_kernel<<<static_cast<unsigned>((out_rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      r->o_acc, r->m, r->l, 1, p->B, p->Hq, p->Sq, static_cast<__nv_bfloat16*>(p->o), p->o_stride_b, p->o_stride_h,
      p->o_stride_s, p->kv_len, r->q_offset, (p->flags & DTB_FLAG_ZERO_PADDED_ROWS) ? 1 : 0);
  return launch_ok("kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}

extern "C" int dtb_fixed_m_operands(const dtb_attn_params* p, float gate, float* norms, float* mk_out, void* stream) {
  int st = check_params(p, false);
  if (st != DTB_OK) return st;
  if (p->flags & DTB_FLAG_QK_FP8) return DTB_ERR_UNSUPPORTED;
  if (norms == nullptr || mk_out == nullptr) return DTB_ERR_NULL;
  if ((reinterpret_cast<uintptr_t>(p->q) & 7u) || (reinterpret_cast<uintptr_t>(p->k) & 7u)) return DTB_ERR_ALIGN;
  // rows are read 8 bytes per lane: every row must start on an 8-byte boundary
  if ((p->q_stride_s & 3) || (p->k_stride_s & 3) || (p->Hq > 1 && (p->q_stride_h & 3)) || (p->Hkv > 1 && (p->k_stride_h & 3)) ||
      (p->B > 1 && ((p->q_stride_b & 3) || (p->k_stride_b & 3))))
    return DTB_ERR_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!cuda_ok(cudaMemsetAsync(norms, 0, sizeof(float) * (p->Hq + p->Hkv), s), "cudaMemsetAsync")) return DTB_ERR_LAUNCH;
  const float scale = p->scale > 0.f ? p->scale : 1.0f / sqrtf(static_cast<float>(p->D));
  // The reference takes the norm of the bf16-rounded product q * scale * log2(e); this kernel
  // applies the scale in f32 after the MMA, so the norm of the unrounded product is the exact bound.
  auto blocks = [](int64_t rows) { return static_cast<unsigned>(std::min<int64_t>((rows + 7) / 8, 148 * 16)); };
  row_norm_max_kernel<<<blocks(static_cast<int64_t>(p->B) * p->Hq * p->Sq), 256, 0, s>>>(
      static_cast<const __nv_bfloat16*>(p->q), p->B, p->Hq, p->Sq, p->q_stride_b, p->q_stride_h, p->q_stride_s,
      scale * kLog2e, norms);
  row_norm_max_kernel<<<blocks(static_cast<int64_t>(p->B) * p->Hkv * p->Skv), 256, 0, s>>>(
      static_cast<const __nv_bfloat16*>(p->k), p->B, p->Hkv, p->Skv, p->k_stride_b, p->k_stride_h, p->k_stride_s, 1.0f,
      norms + p->Hq);
  fixed_m_finish_kernel<<<(p->Hq + 127) / 128, 128, 0, s>>>(norms, p->Hq, p->Hkv, gate, mk_out);
  return launch_ok("kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------------------------
// Split-KV forward for callers that cannot hand over scratch memory.
//
// The partial (o, m, l) states live in a fixed array inside the library image instead of a
// caller-provided workspace.  Every device that loads the library carries the array until the
// process exits.  All calls on a device share it, so two calls whose kernels may overlap on that
// device (different streams, different threads) race on it; callers must order such calls.  Nothing in
// the array needs clearing between calls: the partial kernel writes every (split, row) slot the
// combine kernel reads, empty splits included.
// ---------------------------------------------------------------------------------------------
namespace dtb {
namespace {

static __device__ __align__(256) unsigned char g_static_scratch[DTB_STATIC_SCRATCH_BYTES];

std::mutex g_static_scratch_mu;
void* g_static_scratch_ptr[64] = {};

// Device address of the array on the current device.  In host code `g_static_scratch` is only a
// handle for the runtime, not an address a kernel may use; the address is looked up once per device
// (with that device current) and cached.
int static_scratch_address(void** out) {
  int dev = 0;
  if (!cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return DTB_ERR_LAUNCH;
  if (dev < 0 || dev >= 64) return DTB_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_static_scratch_mu);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    if (!cuda_ok(cudaGetSymbolAddress(&ptr, g_static_scratch), "cudaGetSymbolAddress(static scratch)"))
      return DTB_ERR_LAUNCH;
    if (ptr == nullptr) return DTB_ERR_LAUNCH;
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return DTB_OK;
}

}  // namespace
}  // namespace dtb

extern "C" int dtb_attn_fwd_static_scratch(const dtb_attn_params* p, void* stream) {
  int st = check_params(p, true);
  if (st != DTB_OK) return st;
  if (p->flags & DTB_FLAG_QK_FP8) return DTB_ERR_UNSUPPORTED;
  if (!device_is_sm100()) return DTB_ERR_ARCH;
  const int splits = resolve_splits(p);
  const size_t need = splits > 1 ? split_workspace_bytes(p, splits) : 0;
  if (need > static_cast<size_t>(DTB_STATIC_SCRATCH_BYTES)) {
    char msg[200];
    snprintf(msg, sizeof(msg), "split-KV partials need %zu bytes, the built-in scratch holds %zu", need,
             static_cast<size_t>(DTB_STATIC_SCRATCH_BYTES));
    set_detail(msg);
    return DTB_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  st = static_scratch_address(&scratch);
  if (st != DTB_OK) return st;
  if (!cuda_ok(ensure_kernel_attrs(), "attention kernel attributes (dynamic shared memory size; registers per thread as compiled)")) return DTB_ERR_LAUNCH;
  AttnKernelParams kp;
  st = fill_kernel_params(p, &kp);
  if (st != DTB_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 block(kNumThreads);
  if (splits == 1) {
    attn_fwd_kernel<false, false><<<dim3(q_blocks(p), p->Hq, p->B), block, kSmemBytes, s>>>(kp);
    return launch_ok("attn_fwd_kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
  }
  const size_t rows = static_cast<size_t>(splits) * p->B * p->Hq * p->Sq;
  kp.acc_o = static_cast<float*>(scratch);
  kp.acc_m = kp.acc_o + rows * kHeadDim;
  kp.acc_l = kp.acc_m + rows;
  kp.num_splits = splits;
  kp.acc_init = 1;
  attn_fwd_kernel<true, false><<<dim3(q_blocks(p), p->Hq, p->B * splits), block, kSmemBytes, s>>>(kp);
  if (!launch_ok("attn_fwd_kernel launch")) return DTB_ERR_LAUNCH;
  const int64_t out_rows = static_cast<int64_t>(p->B) * p->Hq * p->Sq;
  combine_kernel<<<static_cast<unsigned>((out_rows + 7) / 8), 256, 0, s>>>(
      kp.acc_o, kp.acc_m, kp.acc_l, splits, p->B, p->Hq, p->Sq, kp.o, kp.o_stride_b, kp.o_stride_h, kp.o_stride_s,
      p->kv_len, 0, kp.zero_padded_rows);
  return launch_ok("combine_kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}

extern "C" int dtb_attn_fwd_scatter(const dtb_attn_params* p, const dtb_attn_scatter* sc, void* stream) {
  int st = check_params(p, false);
  if (st != DTB_OK) return st;
  if (p->flags & DTB_FLAG_QK_FP8) return DTB_ERR_UNSUPPORTED;
  if (sc == nullptr) return DTB_ERR_NULL;
  if (sc->n_peers < 1 || sc->n_peers > 8 || sc->shard_rows <= 0 || sc->total_heads < p->Hq || sc->head_offset < 0 ||
      sc->head_offset + p->Hq > sc->total_heads)
    return DTB_ERR_SHAPE;
  if (static_cast<int64_t>(sc->shard_rows) * sc->n_peers < p->Sq) return DTB_ERR_SHAPE;
  for (int i = 0; i < sc->n_peers; ++i) {
    if (sc->out_ptrs[i] == nullptr) return DTB_ERR_NULL;
    if (reinterpret_cast<uintptr_t>(sc->out_ptrs[i]) & 15u) return DTB_ERR_ALIGN;
  }
  if (!device_is_sm100()) return DTB_ERR_ARCH;
  if (!cuda_ok(ensure_kernel_attrs(), "attention kernel attributes (dynamic shared memory size; registers per thread as compiled)")) return DTB_ERR_LAUNCH;
  AttnKernelParams kp;
  st = fill_kernel_params(p, &kp);
  if (st != DTB_OK) return st;
  for (int i = 0; i < sc->n_peers; ++i) kp.o_peer[i] = static_cast<__nv_bfloat16*>(sc->out_ptrs[i]);
  kp.o_shard_rows = sc->shard_rows;
  kp.o_total_heads = sc->total_heads;
  kp.o_head_offset = sc->head_offset;
  if (p->num_splits == 0 && sc->workspace != nullptr) {
    BalancedPlan plan;
    plan_balanced(p, current_sm_count(), &plan);
    if (plan.use && (reinterpret_cast<uintptr_t>(sc->workspace) & 15u)) return DTB_ERR_ALIGN;
    if (plan.use && sc->workspace_bytes >= balanced_workspace_bytes(plan.slots))
      return launch_balanced(p, kp, plan, sc->workspace, static_cast<cudaStream_t>(stream));
  }
  attn_fwd_kernel<false, false><<<dim3(q_blocks(p), p->Hq, p->B), dim3(kNumThreads), kSmemBytes,
                           static_cast<cudaStream_t>(stream)>>>(kp);
  return launch_ok("attn_fwd_kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}

extern "C" int dtb_scatter_heads(const dtb_scatter_heads_params* sp, void* stream) {
  if (sp == nullptr) return DTB_ERR_NULL;
  if (sp->n_tensors < 1 || sp->n_tensors > 3 || sp->n_peers < 1 || sp->n_peers > 8) return DTB_ERR_SHAPE;
  if (sp->B <= 0 || sp->H <= 0 || sp->S_local <= 0 || sp->D != kHeadDim || sp->H % sp->n_peers != 0 || sp->rank < 0 ||
      sp->rank >= sp->n_peers)
    return DTB_ERR_SHAPE;
  ScatterHeadsParams kp;
  for (int t = 0; t < 3; ++t) {
    const int u = t < sp->n_tensors ? t : 0;
    if (sp->src[u] == nullptr) return DTB_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(sp->src[u]) & 15u) || (sp->stride_b[u] & 7) || (sp->stride_h[u] & 7) || (sp->stride_s[u] & 7))
      return DTB_ERR_ALIGN;
    kp.src[t] = static_cast<const __nv_bfloat16*>(sp->src[u]);
    kp.sb[t] = sp->stride_b[u];
    kp.sh[t] = sp->stride_h[u];
    kp.ss[t] = sp->stride_s[u];
    for (int r = 0; r < 8; ++r) {
      void* d = r < sp->n_peers ? sp->dst[u][r] : nullptr;
      if (r < sp->n_peers && (d == nullptr || (reinterpret_cast<uintptr_t>(d) & 15u))) return d ? DTB_ERR_ALIGN : DTB_ERR_NULL;
      kp.dst[t][r] = static_cast<__nv_bfloat16*>(d);
    }
  }
  kp.B = sp->B;
  kp.H = sp->H;
  kp.Sl = sp->S_local;
  kp.P = sp->n_peers;
  kp.rank = sp->rank;
  const int64_t chunks = static_cast<int64_t>(sp->B) * sp->H * sp->S_local * 16;
  const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((chunks + 255) / 256, 148 * 8));
  scatter_heads_kernel<<<dim3(blocks, sp->n_tensors), 256, 0, static_cast<cudaStream_t>(stream)>>>(kp);
  return launch_ok("scatter_heads_kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}

extern "C" int dtb_attn_fwd_sparse(const dtb_attn_params* p, const dtb_block_table* tb, void* stream) {
  int st = check_params(p, true);
  if (st != DTB_OK) return st;
  if (p->flags & DTB_FLAG_QK_FP8) return DTB_ERR_UNSUPPORTED;
  if (tb == nullptr || tb->kv_table == nullptr || tb->kv_count == nullptr) return DTB_ERR_NULL;
  if (tb->n_classes < 1 || tb->width < 1 || tb->q_blocks != q_blocks(p)) return DTB_ERR_SHAPE;
  if (tb->n_classes > 1 && tb->head_class == nullptr) return DTB_ERR_NULL;
  if (!device_is_sm100()) return DTB_ERR_ARCH;
  if (!cuda_ok(ensure_kernel_attrs(), "attention kernel attributes (dynamic shared memory size; registers per thread as compiled)")) return DTB_ERR_LAUNCH;
  AttnKernelParams kp;
  st = fill_kernel_params(p, &kp);
  if (st != DTB_OK) return st;
  kp.kv_table = tb->kv_table;
  kp.kv_count = tb->kv_count;
  kp.head_class = tb->n_classes > 1 ? tb->head_class : nullptr;
  kp.table_qblocks = tb->q_blocks;
  kp.table_width = tb->width;
  attn_fwd_kernel<false, false><<<dim3(q_blocks(p), p->Hq, p->B), dim3(kNumThreads), kSmemBytes,
                           static_cast<cudaStream_t>(stream)>>>(kp);
  return launch_ok("attn_fwd_kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------------------------
// Saturating E4M3 cast of a bf16 [B, H, S, 128] tensor (values are multiplied by `mult` first, beyond +-448 they
// clamp instead of overflowing), written contiguously.  8 elements per thread.
// ---------------------------------------------------------------------------------------------
namespace dtb {
namespace {
__global__ void __launch_bounds__(256) quantize_e4m3_kernel(const __nv_bfloat16* __restrict__ x, int64_t sb, int64_t sh,
                                                            int64_t ss, int B, int H, int S, float mult,
                                                            uint8_t* __restrict__ out) {
  const int64_t chunks = static_cast<int64_t>(B) * H * S * 16;   // 8 elements each
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < chunks;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx & 15);
    const int64_t rowid = idx >> 4;
    const int s = static_cast<int>(rowid % S);
    const int h = static_cast<int>((rowid / S) % H);
    const int b = static_cast<int>(rowid / (static_cast<int64_t>(S) * H));
    const uint4 raw = reinterpret_cast<const uint4*>(x + b * sb + h * sh + s * ss)[c];
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t packed[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
      f.x *= mult;
      f.y *= mult;
      const uint32_t two = __nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);
      packed[i >> 1] |= two << (16 * (i & 1));
    }
    reinterpret_cast<uint2*>(out + rowid * kHeadDim)[c] = make_uint2(packed[0], packed[1]);
  }
}
}  // namespace
}  // namespace dtb

extern "C" int dtb_quantize_e4m3(const void* x, int64_t stride_b, int64_t stride_h, int64_t stride_s, int32_t B, int32_t H,
                                 int32_t S, int32_t D, float mult, void* out, void* stream) {
  if (x == nullptr || out == nullptr) return DTB_ERR_NULL;
  if (D != kHeadDim || B <= 0 || H <= 0 || S <= 0) return DTB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(out) & 7u) || (stride_b & 7) || (stride_h & 7) ||
      (stride_s & 7))
    return DTB_ERR_ALIGN;
  const int64_t chunks = static_cast<int64_t>(B) * H * S * 16;
  const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((chunks + 255) / 256, 148 * 16));
  quantize_e4m3_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), stride_b, stride_h, stride_s, B, H, S, mult, static_cast<uint8_t*>(out));
  return launch_ok("quantize_e4m3_kernel launch") ? DTB_OK : DTB_ERR_LAUNCH;
}
