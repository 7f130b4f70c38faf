// Joint-attention forward for sm_100a: one CTA owns 256 query rows (two 128-row
// tiles) of one (batch, head) and sweeps the valid keys in 128-key tiles.
//
// Warp roles (384 threads = 3 warpgroups):
//   warps 0-3   softmax group 0: one thread per query row of tile 0
//   warps 4-7   softmax group 1: one thread per query row of tile 1
//   warp  8     MMA issuer (one elected lane issues tcgen05.mma; the warp stays converged)
//   warp  9     TMA producer (lane 0 issues the tensor loads)
//   warps 10-11 idle; they exist so that warps 8-11 form a whole warpgroup, which is the
//               unit setmaxnreg works on: that warpgroup hands registers to the softmax groups
//               (each SM sub-partition holds 16384 registers shared by one warp of each group).
//
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 f32 columns each.  P (bf16)
// is written over the first 64 columns of its S tile (in two halves, each with its
// own mbarrier) and consumed from tensor memory by the PV MMA, so probabilities never
// touch shared memory.
//
// Shared memory: Q (2 x 32 KB, loaded once) and a ring of 32 KB slots through
// which K_0, V_0, K_1, V_1, ... flow; every tile is two 64-column panels written
// by TMA with the 128-byte swizzle the MMA descriptors expect.
//
// The two softmax groups ping-pong: while group 0 exponentiates S0 the tensor
// core runs P1*V and the next Q1*K^T, and vice versa.  MMAs issued by one thread
// execute in order, which is what makes the S/P aliasing and the O rescale safe:
//   * S_t(j+1) = Q_t K_{j+1}^T is issued after O_t += P_t(j) V_j, so it cannot
//     overwrite P_t(j) early;
//   * the commit that publishes S_t(j) follows PV_t(j-1) in issue order, so a
//     softmax thread that has seen S_t(j) may read-modify-write O_t.
#pragma once

#include "ptx.cuh"

namespace dtb {

constexpr int kBlockM = 128;                 // query rows per tile
constexpr int kQTiles = 2;                   // query tiles per CTA
constexpr int kBlockN = 128;                 // keys per tile
constexpr int kHeadDim = 128;
constexpr int kStages = 4;                   // K/V ring slots
constexpr uint32_t kPanelBytes = 128 * 64 * 2;
constexpr uint32_t kTileBytes = 2 * kPanelBytes;
constexpr int kNumSoftmaxThreads = kQTiles * kBlockM;
constexpr int kMmaWarp = kNumSoftmaxThreads / 32;
constexpr int kLoadWarp = kMmaWarp + 1;
constexpr int kNumThreads = kNumSoftmaxThreads + 128;
// Register hand-over between warpgroups.  The kernel is compiled for kLaunchRegs registers per thread (what
// 384 threads can have at most, rounded down to a multiple of 8; the host side refuses to launch a build
// whose count differs).  setmaxnreg.dec in the service warpgroup returns registers to a per-CTA pool and
// setmaxnreg.inc in the two softmax warpgroups takes them from it.  The pool holds nothing else, and an inc
// that asks for more than the decs released waits for ever - no time-out can end that wait - hence the
// static_assert.  (Each sub-partition then holds 2 * 32 * 224 + 32 * 56 = 16128 of its 16384 registers.)
constexpr int kLaunchRegs = 168;
constexpr int kRegsSoftmax = 224;
constexpr int kRegsService = 56;
static_assert((kLaunchRegs - kRegsService) * 128 >= (kRegsSoftmax - kLaunchRegs) * kNumSoftmaxThreads,
              "setmaxnreg.inc would ask for more registers than setmaxnreg.dec releases");
static_assert(kNumThreads * kLaunchRegs <= 65536, "the CTA does not fit the register file");
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;    // log2 units: rescale O only when the row max grew by > 2^8
constexpr float kFixedMRecenter = 88.0f;     // bounded-logit mode exponent offset (m - 88)

struct __align__(8) PipelineBarriers {
  uint64_t q_full[kQTiles];
  uint64_t kv_full[kStages];
  uint64_t kv_empty[kStages];
  uint64_t s_full[kQTiles];
  uint64_t p_lo[kQTiles];   // first 64 keys of P_t written
  uint64_t p_hi[kQTiles];   // last 64 keys of P_t written
  uint64_t o_full[kQTiles];
  uint32_t tmem_base;
  int abort_flag;
};

constexpr size_t kSmemBytes = 1024 /* alignment slack */ + kQTiles * kTileBytes + kStages * kTileBytes +
                              sizeof(PipelineBarriers);

// Barrier-site ids reported in status[1] when a wait runs out.
enum WaitSite : int {
  SITE_Q_FULL = 10, SITE_KV_FULL = 20, SITE_KV_EMPTY = 30, SITE_S_FULL = 40, SITE_P_FULL = 50, SITE_P_HI = 55, SITE_O_FULL = 60
};

struct AttnKernelParams {
  CUtensorMap tmap_q, tmap_k, tmap_v;
  __nv_bfloat16* o;           // normalised output (normal mode)
  int64_t o_stride_b, o_stride_h, o_stride_s;
  float* acc_o;               // residual / partial mode: f32 [units, B, Hq, Sq, D]
  float* acc_m;               //                          f32 [units, B, Hq, Sq]
  float* acc_l;
  const int32_t* kv_len;      // [B] or null
  const float* mk;            // [2, Hq] or null
  int32_t* status;
  int B, Hq, Hkv, Sq, Skv;
  int kv_offset;              // global index of key 0 of this call (ring shards)
  int q_offset;               // global index of query row 0 of this call
  int num_splits;             // >= 1
  int acc_init;               // residual mode: start from the empty state
  int zero_padded_rows;
  float scale_log2;           // softmax scale * log2(e)
  // Head-parallel call with a sequence-sharded output (o_shard_rows > 0): query row s of local head h
  // goes to o_peer[s / o_shard_rows], a contiguous [B, o_total_heads, o_shard_rows, D] buffer that may
  // live on another GPU (plain peer stores), at head o_head_offset + h and row s % o_shard_rows.
  __nv_bfloat16* o_peer[8];
  int o_shard_rows, o_total_heads, o_head_offset;
  // Block-sparse calls (kv_table != null): query block qb of a head in class c visits the key tiles
  // kv_table[(c * table_qblocks + qb) * table_width + i], i < kv_count[c * table_qblocks + qb], ascending.
  const int32_t* kv_table;
  const int32_t* kv_count;
  const int32_t* head_class;   // [Hq] or null (one class)
  int table_qblocks, table_width;
};

// Work list of a balanced launch.  CTAs [0, whole_units) each take one whole (batch, head, query block) unit, in
// unit order (query block fastest).  The units after those - the last, incomplete wave - are cut into pieces of
// nearly equal numbers of key tiles: CTA whole_units + i sweeps key tiles [tile_begin[i], tile_end[i]) of unit
// unit[i] and, unless that is the unit's whole range (slot[i] < 0), leaves its unnormalised (o, m, l) in scratch
// slot slot[i] for the merge kernel.  Pieces are listed longest first, so the hardware's in-order dispatch of
// CTAs to freed SMs packs them evenly.
constexpr int kMaxPieces = 304;
struct PieceTable {
  int whole_units;
  int n_pieces;
  int q_blocks;                      // query blocks per (batch, head): unit = (b * Hq + h) * q_blocks + qblock
  int32_t unit[kMaxPieces];
  uint16_t tile_begin[kMaxPieces];
  uint16_t tile_end[kMaxPieces];
  int16_t slot[kMaxPieces];
};

// Warp-uniform bounded wait: every lane polls, and the warp agrees on the outcome so
// that warp-collective instructions after it are never reached by a partial warp.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, const AbortCtx& ctx, int site) {
  return __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), parity, ctx, site));
}

// ---------------------------------------------------------------------------
// One key tile of softmax for the row owned by this thread.
//
// The whole S row comes out of tensor memory in one load; the row max uses three-input max; the
// scale-and-subtract and the row sum run on packed f32 pairs; P goes back to tensor memory in two
// halves of 64 keys, each published on its own mbarrier so the PV MMA of the first half runs while
// the second half is still being exponentiated.  Once the rows have an offset, the first half is exponentiated
// with it before the row max is known (see below): the max then only confirms that the offset can stay.
// ---------------------------------------------------------------------------
template <bool kFixedM>
__device__ __forceinline__ void softmax_tile(uint32_t s_tmem, uint32_t o_tmem, float scale_log2, int valid_cols,
                                             bool o_live, float& m_used, float& l_sum, uint32_t bar_p_lo,
                                             uint32_t bar_p_hi) {
  uint32_t sr[kBlockN];
  tmem_ld128_sync(s_tmem, sr);
  if (valid_cols < kBlockN) {
#pragma unroll
    for (int i = 0; i < kBlockN; ++i)
      if (i >= valid_cols) sr[i] = 0xff800000u;  // -inf
  }
  const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2);
  uint64_t acc2 = pack_f32x2(0.f, 0.f);
  uint32_t pk[32];
  // 2^(s * scale - m) for 64 keys: packed into pk, summed into acc2.
  auto exp_half = [&](int half, float m) {
    const uint64_t neg_m2 = pack_f32x2(-m, -m);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int col = half * 64 + 2 * i;
      const uint64_t x2 = fma_f32x2(pack_f32x2(__uint_as_float(sr[col]), __uint_as_float(sr[col + 1])), scale2, neg_m2);
      float x0, x1, p0, p1;
      unpack_f32x2(x2, x0, x1);
      p0 = ex2(x0);
      p1 = ex2(x1);
      acc2 = add_f32x2(acc2, pack_f32x2(p0, p1));
      pk[i] = pack_bf16x2(p0, p1);
      // The first 32 keys of the half go to tensor memory while the other 32 are exponentiated, which hides half
      // of the store's latency.  Nothing reads them before the arrive in publish(), so a speculated half that is
      // thrown away is simply overwritten.
      if (i == 15) tmem_st16(s_tmem + half * 32, pk);
    }
  };
  auto publish = [&](int half) {
    tmem_st16(s_tmem + half * 32 + 16, pk + 16);
    tmem_wait_st();
    tc_fence_before();
    mbar_arrive(half == 0 ? bar_p_lo : bar_p_hi);
  };
  auto finish = [&]() {
    float a0, a1;
    unpack_f32x2(acc2, a0, a1);
    l_sum += a0 + a1;
  };
  // The row maximum in log2 units: eight independent chains of three-input max keep the dependency depth at 8 + 3.
  auto row_max = [&]() {
    float mxs[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) mxs[c] = fmaxf(__uint_as_float(sr[c]), __uint_as_float(sr[c + 8]));
#pragma unroll
    for (int i = 16; i < kBlockN; i += 16) {
#pragma unroll
      for (int c = 0; c < 8; ++c) mxs[c] = max3(mxs[c], __uint_as_float(sr[i + c]), __uint_as_float(sr[i + c + 8]));
    }
    return fmaxf(max3(mxs[0], mxs[1], mxs[2]), fmaxf(max3(mxs[3], mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7]))) * scale_log2;
  };

  if (!kFixedM) {
    // The maximum only decides whether the offset in use has to move, which after the first tiles is rare
    // (kRescaleThreshold).  So once every row of the warp has an offset, the first half of P is exponentiated with
    // it in the same straight-line code as the reduction of the maximum - the exponentials wait on the MUFU unit,
    // the maxima fill the issue slots between them - and that work is thrown away only if some row does move.
    // On the 1024-pixel image shape this takes a call from 398 to 390 us.
    if (__all_sync(0xffffffffu, m_used > -INFINITY)) {
      exp_half(0, m_used);
      const float mx = row_max();
      if (!__any_sync(0xffffffffu, mx > m_used + kRescaleThreshold)) {
        publish(0);
        exp_half(1, m_used);
        publish(1);
        finish();
        return;
      }
      acc2 = pack_f32x2(0.f, 0.f);
      tmem_wait_st();   // the speculated store has to land before the same columns are written again
    }
    const float mx = row_max();
    const bool grow = mx > m_used + kRescaleThreshold;  // always true while m_used == -inf
    if (o_live && __any_sync(0xffffffffu, grow)) {
      const float alpha = grow ? ex2(m_used - mx) : 1.0f;
      l_sum *= alpha;
      uint32_t r[32];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tmem_ld32_sync(o_tmem + c * 32, r);
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
        tmem_st32(o_tmem + c * 32, r);
      }
    } else if (grow) {
      // No accumulator yet: only the running sum carries history (it is 0 or, in
      // residual mode with an empty incoming state, already 0).
      l_sum *= ex2(m_used - mx);
    }
    if (grow) m_used = mx;
  }
  exp_half(0, m_used);
  publish(0);
  exp_half(1, m_used);
  publish(1);
  finish();
}

// ---------------------------------------------------------------------------
// The kernel.  kResidual = false: write the normalised bf16 output.
//              kResidual = true : fold into / emit the running (o, m, l) state
//                                 (ring steps and split-KV partials).
// ---------------------------------------------------------------------------
//              kQkFp8 = true    : q and k are E4M3 bytes ([B, H, S, 128] with byte strides); the score MMA runs as
//                                 kind::f8f6f4 with 32 contraction elements per instruction, P*V stays bf16.
//              kTable = true    : the CTA's work comes from a PieceTable (balanced launch); a piece that covers only
//                                 part of a unit's keys emits its state like a residual call, a whole unit
//                                 writes the normalised output.
template <bool kResidual, bool kQkFp8, bool kTable>
__device__ __forceinline__ void attn_fwd_body(const AttnKernelParams& p, const PieceTable* tb) {
  constexpr uint32_t kQkTileBytes = kQkFp8 ? kPanelBytes : kTileBytes;   // bytes of one 128-row Q or K tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem;
  {
    const uint32_t a = smem_u32(smem_raw);
    smem = smem_raw + (((a + 1023u) & ~1023u) - a);
  }
  uint8_t* smem_q = smem;
  uint8_t* smem_kv = smem + kQTiles * kTileBytes;
  PipelineBarriers* bars = reinterpret_cast<PipelineBarriers*>(smem_kv + kStages * kTileBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int split = 0, b, h, qblock, piece_begin = 0, piece_end = 0x7fffffff, slot = -1;
  if (kTable) {
    const int id = blockIdx.x;
    int unit_id = id;
    if (id >= tb->whole_units) {
      const int i = id - tb->whole_units;
      unit_id = tb->unit[i];
      piece_begin = tb->tile_begin[i];
      piece_end = tb->tile_end[i];
      slot = tb->slot[i];
    }
    qblock = unit_id % tb->q_blocks;
    const int bh = unit_id / tb->q_blocks;
    h = bh % p.Hq;
    b = bh / p.Hq;
  } else {
    split = blockIdx.z % p.num_splits;
    b = blockIdx.z / p.num_splits;
    h = blockIdx.y;
    qblock = blockIdx.x;
  }
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qblock * (kQTiles * kBlockM);
  const bool emit_state = kResidual || (kTable && slot >= 0);   // leave (o, m, l) instead of the normalised output

  // Valid keys of this call: global indices [kv_offset, kv_offset + Skv) below kv_len[b].
  const int kv_len_b = (p.kv_len != nullptr) ? max(p.kv_len[b], 0) : 0x7fffffff;
  const int kv_eff = max(min(kv_len_b - p.kv_offset, p.Skv), 0);
  // Key tiles this query block visits: all of [0, ceil(kv_eff / 128)) or, for a block-sparse call, the
  // entries of its table row that start below kv_eff (the row is ascending: binary search).
  const int32_t* tile_list = nullptr;
  int n_total = (kv_eff + kBlockN - 1) / kBlockN;
  if (p.kv_table != nullptr) {
    const int cls = p.head_class != nullptr ? p.head_class[h] : 0;
    const int64_t trow = static_cast<int64_t>(cls) * p.table_qblocks + qblock;
    tile_list = p.kv_table + trow * p.table_width;
    int lo = 0, hi = p.kv_count[trow];
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (tile_list[mid] * kBlockN < kv_eff) lo = mid + 1; else hi = mid;
    }
    n_total = lo;
  }
  const int per_split = (n_total + p.num_splits - 1) / p.num_splits;
  const int tile_begin = kTable ? min(piece_begin, n_total) : min(split * per_split, n_total);
  const int tile_end = kTable ? min(piece_end, n_total) : min(tile_begin + per_split, n_total);
  const int n_tiles = tile_end - tile_begin;
  const bool block_padded = p.zero_padded_rows && (p.q_offset + q0 >= kv_len_b);

  // first row of this CTA's (o, m, l) rows in the state arrays, minus q0 (so that + row addresses them)
  const int64_t unit = kResidual ? ((static_cast<int64_t>(split) * p.B + b) * p.Hq + h) : 0;
  const int64_t acc_base = kTable ? static_cast<int64_t>(slot) * (kQTiles * kBlockM) - q0 : unit * p.Sq;

  if (n_tiles <= 0 || block_padded) {
    // Nothing to attend to: emit zeros (normal) or the empty state (residual, when initialising).
    if (threadIdx.x < kNumSoftmaxThreads) {
      const int row = q0 + threadIdx.x;
      if (row < p.Sq) {
        if (!emit_state) {
          uint4* dst;
          if (p.o_shard_rows > 0) {
            const int dest = row / p.o_shard_rows;
            dst = reinterpret_cast<uint4*>(
                p.o_peer[dest] + ((static_cast<int64_t>(b) * p.o_total_heads + p.o_head_offset + h) * p.o_shard_rows +
                                  (row - dest * p.o_shard_rows)) * kHeadDim);
          } else {
            dst = reinterpret_cast<uint4*>(p.o + b * p.o_stride_b + h * p.o_stride_h + row * p.o_stride_s);
          }
#pragma unroll
          for (int i = 0; i < kHeadDim * 2 / 16; ++i) dst[i] = make_uint4(0, 0, 0, 0);
        } else if (p.acc_init) {
          float4* dst = reinterpret_cast<float4*>(p.acc_o + (acc_base + row) * kHeadDim);
#pragma unroll
          for (int i = 0; i < kHeadDim / 4; ++i) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          p.acc_m[acc_base + row] = -INFINITY;
          p.acc_l[acc_base + row] = 0.f;
        }
      }
    }
    return;
  }

  AbortCtx ctx{&bars->abort_flag, p.status};

  if (threadIdx.x == kMmaWarp * 32) {
    bars->abort_flag = 0;
    for (int i = 0; i < kQTiles; ++i) {
      mbar_init(smem_u32(&bars->q_full[i]), 1);
      mbar_init(smem_u32(&bars->s_full[i]), 1);
      mbar_init(smem_u32(&bars->p_lo[i]), kBlockM);
      mbar_init(smem_u32(&bars->p_hi[i]), kBlockM);
      mbar_init(smem_u32(&bars->o_full[i]), 1);
    }
    for (int i = 0; i < kStages; ++i) {
      mbar_init(smem_u32(&bars->kv_full[i]), 1);
      mbar_init(smem_u32(&bars->kv_empty[i]), 1);
    }
    mbar_fence_init();
  }
  if (warp == kLoadWarp && lane == 0) {
    tma_prefetch_desc(&p.tmap_q);
    tma_prefetch_desc(&p.tmap_k);
    tma_prefetch_desc(&p.tmap_v);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&bars->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == kLoadWarp) {
    // ------------------------------------------------------------------ TMA producer
    setmaxnreg_dec<kRegsService>();
    bool ok = true;
    if (lane == 0) {
      for (int t = 0; t < kQTiles; ++t) {
        const uint32_t bar = smem_u32(&bars->q_full[t]);
        mbar_expect_tx(bar, kQkTileBytes);
        const uint32_t dst = smem_u32(smem_q + t * kTileBytes);
        tma_load_4d(dst, &p.tmap_q, bar, 0, q0 + t * kBlockM, h, b);
        if (!kQkFp8) tma_load_4d(dst + kPanelBytes, &p.tmap_q, bar, 64, q0 + t * kBlockM, h, b);
      }
      for (int i = 0; i < 2 * n_tiles && ok; ++i) {
        const int slot = i % kStages;
        const int use = i / kStages;
        if (use > 0) ok = mbar_wait(smem_u32(&bars->kv_empty[slot]), (use - 1) & 1, ctx, SITE_KV_EMPTY + slot);
        if (!ok) break;
        const uint32_t bar = smem_u32(&bars->kv_full[slot]);
        const bool is_v = (i & 1) != 0;
        mbar_expect_tx(bar, is_v ? kTileBytes : kQkTileBytes);
        const uint32_t dst = smem_u32(smem_kv + slot * kTileBytes);
        const int entry = tile_begin + (i >> 1);
        const int row = (tile_list != nullptr ? tile_list[entry] : entry) * kBlockN;
        const CUtensorMap* tm = is_v ? &p.tmap_v : &p.tmap_k;
        tma_load_4d(dst, tm, bar, 0, row, hk, b);
        if (is_v || !kQkFp8) tma_load_4d(dst + kPanelBytes, tm, bar, 64, row, hk, b);
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    setmaxnreg_dec<kRegsService>();
    constexpr uint32_t idesc_qk = kQkFp8 ? make_idesc_e4m3(kBlockM, kBlockN) : make_idesc_bf16(kBlockM, kBlockN, false, false);
    constexpr uint32_t idesc_pv = make_idesc_bf16(kBlockM, kHeadDim, false, true);
    const uint64_t q_desc0 = make_smem_desc_sw128(smem_u32(smem_q), 16, 1024);
    const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(smem_kv), 16, 1024);
    const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(smem_kv), kPanelBytes, 1024);
    bool ok = true;

    // The issuing regions are entered through elect.sync rather than `lane == 0`: with the same instructions inside,
    // a call on the 1024-pixel image shape takes 399 us against 413 us.  Everything this warp does between two MMA
    // instructions is idle time of the tensor pipe, so the code the compiler emits around them matters.
    auto issue_qk = [&](int t, int slot) {
      if (elect_one()) {
        const uint64_t a0 = q_desc0 + static_cast<uint64_t>((t * kTileBytes) >> 4);
        const uint64_t b0 = k_desc0 + static_cast<uint64_t>((slot * kTileBytes) >> 4);
        if (kQkFp8) {
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 32; ++kk) {   // 32 one-byte elements = 32 bytes of the swizzled row
            const uint64_t off = static_cast<uint64_t>((kk * 32) >> 4);
            mma_ss_f8(tmem_base + t * kBlockN, a0 + off, b0 + off, idesc_qk, kk > 0 ? 1u : 0u);
          }
        } else {
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk) {
            const uint64_t off = static_cast<uint64_t>(((kk & 3) * 32 + (kk >> 2) * kPanelBytes) >> 4);
            mma_ss(tmem_base + t * kBlockN, a0 + off, b0 + off, idesc_qk, kk > 0 ? 1u : 0u);
          }
        }
        mma_commit(smem_u32(&bars->s_full[t]));
      }
      __syncwarp();
    };
    auto issue_pv = [&](int t, int slot, int half, bool accumulate) {
      if (elect_one()) {
        const uint64_t b0 = v_desc0 + static_cast<uint64_t>((slot * kTileBytes) >> 4);
        const uint32_t d_tmem = tmem_base + (kQTiles + t) * kBlockN;
        const uint32_t a_tmem = tmem_base + t * kBlockN;
#pragma unroll
        for (int kk = half * 4; kk < half * 4 + 4; ++kk) {
          const uint64_t off = static_cast<uint64_t>((kk * 16 * 128) >> 4);
          mma_ts(d_tmem, a_tmem + kk * 8, b0 + off, idesc_pv, (accumulate || kk > 0) ? 1u : 0u);
        }
      }
      __syncwarp();
    };
    auto commit_to = [&](uint64_t* bar) {
      if (elect_one()) mma_commit(smem_u32(bar));
      __syncwarp();
    };
    auto wait_kv = [&](int i) {
      const int slot = i % kStages;
      return warp_wait(&bars->kv_full[slot], (i / kStages) & 1, ctx, SITE_KV_FULL + slot);
    };

    // Prologue: S_t(0) = Q_t K_0^T for both tiles.
    ok = warp_wait(&bars->q_full[0], 0, ctx, SITE_Q_FULL);
    if (ok) ok = wait_kv(0);
    if (ok) {
      tc_fence_after();
      issue_qk(0, 0);
      ok = warp_wait(&bars->q_full[1], 0, ctx, SITE_Q_FULL + 1);
    }
    if (ok) {
      tc_fence_after();
      issue_qk(1, 0);
      commit_to(&bars->kv_empty[0]);
    }
    const bool o_preloaded = kResidual && !p.acc_init;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int iv = 2 * j + 1;
      const int ik = 2 * j + 2;
      // No wait for V_j or K_{j+1} here: softmax group 0 checks both loads before it publishes P_0(j) (see
      // there), so the P barriers below already say that the tiles have landed.
      for (int t = 0; t < kQTiles && ok; ++t) {
        ok = warp_wait(&bars->p_lo[t], j & 1, ctx, SITE_P_FULL + t);
        if (!ok) break;
        tc_fence_after();
        issue_pv(t, iv % kStages, 0, j > 0 || o_preloaded);
        ok = warp_wait(&bars->p_hi[t], j & 1, ctx, SITE_P_HI + t);
        if (!ok) break;
        tc_fence_after();
        issue_pv(t, iv % kStages, 1, true);
        if (t == kQTiles - 1) commit_to(&bars->kv_empty[iv % kStages]);
        if (j + 1 < n_tiles) {
          issue_qk(t, ik % kStages);
          if (t == kQTiles - 1) commit_to(&bars->kv_empty[ik % kStages]);
        } else {
          commit_to(&bars->o_full[t]);
        }
      }
    }
  } else if (warp < kMmaWarp) {
    // ------------------------------------------------------------------ softmax groups
    setmaxnreg_inc<kRegsSoftmax>();
    const int t = warp >> 2;                       // query tile of this group
    const int row_in_tile = threadIdx.x & (kBlockM - 1);
    const int row = q0 + t * kBlockM + row_in_tile;  // query row within this call
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_off + t * kBlockN;
    const uint32_t o_tmem = tmem_base + lane_off + (kQTiles + t) * kBlockN;
    const float scale_log2 = p.scale_log2;
    const bool row_in_range = row < p.Sq;
    const int64_t acc_row = acc_base + row;
    const uint32_t bar_p_lo = smem_u32(&bars->p_lo[t]);
    const uint32_t bar_p_hi = smem_u32(&bars->p_hi[t]);

    float m_used = -INFINITY;
    float l_sum = 0.f;
    bool fixed_m = false;
    if (p.mk != nullptr && p.mk[p.Hq + h] > 0.5f) {
      fixed_m = true;
      m_used = p.mk[h] - kFixedMRecenter;
    }
    bool o_live = false;
    if (kResidual && !p.acc_init) {
      // Bring the running state of this row into registers / tensor memory.
      float m_in = -INFINITY, l_in = 0.f;
      if (row_in_range) {
        m_in = p.acc_m[acc_row];
        l_in = p.acc_l[acc_row];
      }
      const float4* src = reinterpret_cast<const float4*>(p.acc_o + acc_row * kHeadDim);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float4 v = row_in_range ? src[c * 8 + i] : make_float4(0.f, 0.f, 0.f, 0.f);
          r[4 * i] = __float_as_uint(v.x);
          r[4 * i + 1] = __float_as_uint(v.y);
          r[4 * i + 2] = __float_as_uint(v.z);
          r[4 * i + 3] = __float_as_uint(v.w);
        }
        tmem_st32(o_tmem + c * 32, r);
      }
      tmem_wait_st();
      o_live = true;
      if (fixed_m) {
        // The incoming state is expressed relative to m_in; re-express it relative to the fixed offset.
        // (Callers that use the bounded-logit mode keep one offset for the whole ring, so this is a no-op.)
        const bool shift = (m_in != m_used) && (l_in > 0.f);
        if (__any_sync(0xffffffffu, shift)) {
          const float alpha = shift ? ex2(m_in - m_used) : 1.0f;
          l_in *= alpha;
          uint32_t r[32];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            tmem_ld32_sync(o_tmem + c * 32, r);
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(o_tmem + c * 32, r);
          }
          tmem_wait_st();
        }
      } else {
        m_used = m_in;
      }
      l_sum = l_in;
    }

    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      // The MMA issuer pays ~100 cycles of idle tensor pipe for every barrier it polls, even a satisfied one,
      // while this group spends a third of every iteration waiting for S.  So one thread of group 0 checks here
      // that V_j and K_{j+1} have landed (they were requested two tiles ago); its arrival on the P barriers then
      // carries that fact to the issuer, which uses V_j first in P_0(j) V_j and K_{j+1} first in Q_0 K_{j+1}^T.
      bool kv_ok = true;
      if (threadIdx.x == 0) {
        const int iv = 2 * j + 1, ik = 2 * j + 2;
        kv_ok = mbar_wait(smem_u32(&bars->kv_full[iv % kStages]), (iv / kStages) & 1, ctx, SITE_KV_FULL + iv % kStages);
        if (kv_ok && j + 1 < n_tiles)
          kv_ok = mbar_wait(smem_u32(&bars->kv_full[ik % kStages]), (ik / kStages) & 1, ctx, SITE_KV_FULL + ik % kStages);
      }
      ok = __all_sync(0xffffffffu, kv_ok && mbar_wait(smem_u32(&bars->s_full[t]), j & 1, ctx, SITE_S_FULL + t));
      if (!ok) break;
      tc_fence_after();
      const int tile = tile_list != nullptr ? tile_list[tile_begin + j] : tile_begin + j;
      const int valid_cols = min(kv_eff - tile * kBlockN, kBlockN);
      if (fixed_m) {
        softmax_tile<true>(s_tmem, o_tmem, scale_log2, valid_cols, o_live, m_used, l_sum, bar_p_lo, bar_p_hi);
      } else {
        softmax_tile<false>(s_tmem, o_tmem, scale_log2, valid_cols, o_live, m_used, l_sum, bar_p_lo, bar_p_hi);
      }
      o_live = true;
    }
    if (ok) ok = warp_wait(&bars->o_full[t], 0, ctx, SITE_O_FULL + t);
    if (ok) {
      tc_fence_after();
      if (emit_state) {
        float4* dst = reinterpret_cast<float4*>(p.acc_o + acc_row * kHeadDim);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32_sync(o_tmem + c * 32, r);
          if (row_in_range) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              dst[c * 8 + i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                           __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
          }
        }
        if (row_in_range) {
          p.acc_m[acc_row] = m_used;
          p.acc_l[acc_row] = l_sum;
        }
      } else {
        // Normalise, round to bf16 and stage the 32 rows of this warp in the (now dead) Q tile of
        // this group, 16-byte chunks XOR-swizzled by row so neither side bank-conflicts; then the warp
        // writes whole 256-byte rows, two per store instruction, to this GPU's output or, for a
        // head-parallel call whose output is sequence-sharded, straight into the owning peer's buffer.
        const bool padded = p.zero_padded_rows && (p.q_offset + row >= kv_len_b);
        const float inv = (l_sum > 0.f && !padded) ? (1.0f / l_sum) : 0.f;
        uint8_t* stage = smem_q + t * kTileBytes + (warp & 3) * (32 * kHeadDim * 2);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32_sync(o_tmem + c * 32, r);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * i]) * inv, __uint_as_float(r[8 * i + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv);
            const int chunk = c * 4 + i;
            *reinterpret_cast<uint4*>(stage + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = v;
          }
        }
        __syncwarp();
        const int row0 = q0 + t * kBlockM + (warp & 3) * 32;   // first query row of this warp
        const int sub = lane >> 4;                              // which of the two rows of a store
        const int chunk = lane & 15;
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
          const int rl = 2 * i + sub;
          const int grow = row0 + rl;
          if (grow < p.Sq) {
            const uint4 v = *reinterpret_cast<const uint4*>(stage + rl * 256 + ((chunk ^ (rl & 15)) << 4));
            __nv_bfloat16* dst_row;
            if (p.o_shard_rows > 0) {
              const int dest = grow / p.o_shard_rows;
              dst_row = p.o_peer[dest] +
                        ((static_cast<int64_t>(b) * p.o_total_heads + p.o_head_offset + h) * p.o_shard_rows +
                         (grow - dest * p.o_shard_rows)) * kHeadDim;
            } else {
              dst_row = p.o + b * p.o_stride_b + h * p.o_stride_h + grow * p.o_stride_s;
            }
            reinterpret_cast<uint4*>(dst_row)[chunk] = v;
          }
        }
      }
    }
  }

  else {
    setmaxnreg_dec<kRegsService>();  // idle warps of the service warpgroup
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (bars->abort_flag) {
    // Give copies and MMAs that are still in flight time to land before the
    // shared and tensor memory they target is released.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

template <bool kResidual, bool kQkFp8>
__global__ void __launch_bounds__(kNumThreads, 1) attn_fwd_kernel(const __grid_constant__ AttnKernelParams p) {
  attn_fwd_body<kResidual, kQkFp8, false>(p, nullptr);
}

// The balanced launch of the plain bf16 forward: a 1-D grid of whole units followed by the pieces of `tb`.
__global__ void __launch_bounds__(kNumThreads, 1) attn_fwd_pieces_kernel(const __grid_constant__ AttnKernelParams p,
                                                                         const __grid_constant__ PieceTable tb) {
  attn_fwd_body<false, false, true>(p, &tb);
}

}  // namespace dtb
