// Backward without atomics: one streaming kernel in two modes, launched one after the other.
//
//   mode dK/dV (kDKV = true):  a work item is one (batch, head, 128-key tile).  K_j, V_j stay in shared
//       memory, dK_j, dV_j in TMEM, and the query side (Q_i, dO_i) is streamed past them.
//   mode dQ    (kDKV = false): a work item is one (batch, head, 128-query tile).  Q_i, dO_i stay in shared
//       memory, dQ_i in TMEM, and the key side (K_j, V_j) is streamed past them.
//
// This is the split of the reference's backward (_bwd_dense_dkdv_kernel and _bwd_dense_dq_kernel,
// src/triton_sigmoid/sigmoid_triton_dense.py:315-467 and 162-307; padded pair
// src/triton_sigmoid/sigmoid_triton_padded.py:342-509 and 179-339): S and dP are computed in both modes
// (7 GEMMs per tile pair in total), and in exchange nothing is accumulated across CTAs: no fp32 workspace,
// no reductions through the L2, no conversion pass, and run-to-run deterministic gradients.  (The fused
// 5-GEMM kernel in bwd_kernel.cuh pays for its two saved GEMMs with fp32 reductions of dQ whose L2
// traffic bounds it.)
//
// With R = the stationary ("row") side and C = the streamed ("column") side, both modes are
//     S   = R1 C1^T     (K Q^T   | Q K^T)      smem x smem -> TMEM fp32, N = 64 columns per job
//     dP  = R2 C2^T     (V dO^T  | dO V^T)
//     P   = sigmoid(scale S + bias),  dS = P (1 - P) dP                 (registers)
//     out1 += dS C1     (dK += dS^T Q | dQ += dS K)   TMEM(16-bit) x smem -> TMEM fp32
//     out2 += P  C2     (dV += P^T dO | -)            dK/dV mode only
// A JOB is the row tile times 64 columns of the streamed side; its S and dP share a 128-column TMEM slot
// (ring of 3; 2 for dK/dV at D = 128), P and dS are written over the columns they were computed from.
//
// Warp roles (20 warps): 0-15 compute warps in two groups of eight that take jobs alternately (warp w:
// TMEM lanes 32 (w & 3).., columns 32 ((w >> 2) & 1).. of the job); 16 item scheduler + TMA producer;
// 17 issuer of S and dP (owns the TMEM allocation); 18 issuer of out1 / out2; 19 idle.
#pragma once

#include "ptx.cuh"
#include "sigmoid_math.cuh"

namespace sigattn {

struct BwdStreamParams {
  void* out1;  // dK (dK/dV mode) or dQ (dQ mode): rows of the stationary side
  void* out2;  // dV (dK/dV mode only)
  int64_t o1_sb, o1_st, o1_sh;
  int64_t o2_sb, o2_st, o2_sh;
  const int* lens_r;  // valid lengths of the stationary side (keys in dK/dV mode, queries in dQ mode) or nullptr
  const int* lens_c;  // valid lengths of the streamed side
  const int* cu_r;    // packed layout: row offsets of the stationary side / streamed side, or nullptr
  const int* cu_c;
  const float* bias;       // [B] or nullptr
  const float* score_mod;  // per (batch, key) or nullptr
  float scale;
  float bias_scalar;
  int B, H, Tr, Tc;  // extents of the stationary and the streamed side
  int Tk;            // key extent (row length of score_mod)
  int causal;
  int n_rblk;   // ceil(Tr / 128)
  int n_items;  // B * H * n_rblk
  int group;    // (batch, head) pairs per scheduling group
  unsigned int* ticket;
};

constexpr int kBsComputeWarps = 16;
constexpr int kBsGroupWarps = 8;
constexpr int kBsProducerWarp = 16;
constexpr int kBsIssuerIn = 17;   // S, dP; owns the TMEM allocation
constexpr int kBsIssuerOut = 18;  // out1, out2
constexpr int kBsThreads = 20 * 32;
constexpr int kBsTile = 128;
constexpr int kBsJobN = 64;

template <int D, bool kDKV>
struct BsSmem {
  static constexpr int kStages = (D == 64) ? 3 : 2;       // streamed (C1, C2) tile pairs
  static constexpr int kRBufs = (D == 64) ? 2 : 1;        // stationary (R1, R2) tile pairs
  static constexpr int kSlots = (kDKV && D == 128) ? 2 : 3;
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kR1Off = 0;
  static constexpr int kR2Off = kR1Off + kRBufs * kTileBytes;
  static constexpr int kC1Off = kR2Off + kRBufs * kTileBytes;
  static constexpr int kC2Off = kC1Off + kStages * kTileBytes;
  static constexpr int kBarOff = kC2Off + kStages * kTileBytes;
  static constexpr int kRFull = 0;                     // [2] per R buffer (both tiles)
  static constexpr int kREmpty = kRFull + 2;           // [2] every S / dP product that reads the buffer is complete
  static constexpr int kCFull = kREmpty + 2;           // [kStages] both streamed tiles of the stage
  static constexpr int kCEmpty = kCFull + kStages;     // [kStages] both issuers have finished with the stage
  static constexpr int kCFix = kCEmpty + kStages;      // [kStages] rows beyond the valid length zeroed
  static constexpr int kInFull = kCFix + kStages;      // [kSlots] S and dP of the slot's job complete
  static constexpr int kOutReady = kInFull + kSlots;   // [kSlots] P / dS written (8 warps)
  static constexpr int kSlotFree = kOutReady + kSlots; // [kSlots] out products of the slot's job complete
  static constexpr int kAccFull = kSlotFree + kSlots;  // every product of the item complete
  static constexpr int kAccEmpty = kAccFull + 1;       // accumulators read out of TMEM (16 warps)
  static constexpr int kItemFull = kAccEmpty + 1;      // [2]
  static constexpr int kItemEmpty = kItemFull + 2;     // [2]
  static constexpr int kNumBars = kItemEmpty + 2;
  static constexpr int kMiscOff = kBarOff + 8 * kNumBars;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynBytes = kTotal + 1024;
};

// One work item, decoded the same way by every warp role.
struct BsItem {
  int b, h, r0;       // first row of the stationary tile within its sequence
  int bc;             // batch coordinate of the tensor maps and strides (0 when packed)
  int tr0, tc0;       // first row of the sequence on the stationary / streamed side (0 unless packed)
  int tk0;            // first key of the sequence (for score_mod)
  int row_lim;        // rows below this exist in this sequence's tensors
  int Lr, Lc;
  int hj_begin, hj_end;  // 64-column jobs [hj_begin, hj_end) of the streamed side
  int n_jobs;
};
template <bool kDKV>
__device__ __forceinline__ BsItem bs_decode_item(const BwdStreamParams& p, int item) {
  BsItem it;
  // Groups of `group` (batch, head) pairs; within a group the heavy row tiles of all pairs come first
  // (under a causal mask: early key tiles in dK/dV mode, late query tiles in dQ mode).
  const int per_group = p.group * p.n_rblk;
  const int grp = item / per_group;
  const int r = item - grp * per_group;
  const int g_eff = min(p.group, p.B * p.H - grp * p.group);
  const int ri = r / g_eff;
  const int bh = grp * p.group + (r - ri * g_eff);
  it.b = bh / p.H;
  it.h = bh - it.b * p.H;
  const int rblk = (!kDKV && p.causal) ? (p.n_rblk - 1 - ri) : ri;
  it.r0 = rblk * kBsTile;
  it.Lr = p.Tr;
  it.Lc = p.Tc;
  if (p.lens_r) it.Lr = min(max(p.lens_r[it.b], 0), p.Tr);
  if (p.lens_c) it.Lc = min(max(p.lens_c[it.b], 0), p.Tc);
  it.bc = it.b;
  it.tr0 = it.tc0 = 0;
  it.row_lim = p.Tr;
  if (p.cu_r) {
    it.tr0 = p.cu_r[it.b];
    it.tc0 = p.cu_c[it.b];
    it.Lr = min(max(p.cu_r[it.b + 1] - it.tr0, 0), p.Tr);
    it.Lc = min(max(p.cu_c[it.b + 1] - it.tc0, 0), p.Tc);
    it.bc = 0;
    it.row_lim = it.Lr;
  }
  it.tk0 = kDKV ? it.tr0 : it.tc0;
  if (kDKV) {
    // keys [r0, r0+128) are seen by queries >= r0 (causal, top-left aligned) and < Lq
    it.hj_begin = p.causal ? (it.r0 / kBsJobN) : 0;
    it.hj_end = (it.Lc + kBsJobN - 1) / kBsJobN;
  } else {
    // queries [r0, r0+128) see keys < Lk and <= their own index
    it.hj_begin = 0;
    const int c_end = p.causal ? min(it.Lc, it.r0 + kBsTile) : it.Lc;
    it.hj_end = (c_end + kBsJobN - 1) / kBsJobN;
  }
  it.n_jobs = (it.r0 < it.Lr) ? max(it.hj_end - it.hj_begin, 0) : 0;
  return it;
}

// 16 score columns and 16 dP columns of one TMEM lane -> P (kept for the caller in 16-bit pairs when
// kStoreP) and dS = P (1 - P) dP, both written back over the first 8 of the columns they came from.
// Valid columns for this lane are [lo, hi) (used only when kMask); col0 = index of the first column.
template <bool kBF16, bool kStoreP, bool kMask, bool kAccurate>
__device__ __forceinline__ void bs_unit16(uint32_t s_addr, uint32_t dp_addr, const uint32_t (&rs)[16],
                                          const uint32_t (&rd)[16], float c1, float c0, int col0, int lo, int hi,
                                          const float* mod_cols, int mod_lim) {
  float2 t[8];
  constexpr bool kShift = !kMask && !kAccurate;
  const float c0s = kShift ? c0 + kDeepShift : c0;
#pragma unroll
  for (int i = 0; i < 8; ++i)
    t[i] = __ffma2_rn(make_float2(__uint_as_float(rs[2 * i]), __uint_as_float(rs[2 * i + 1])), make_float2(c1, c1),
                      make_float2(c0s, c0s));
  if (mod_cols) {
    // per-key additive bias along the columns (dQ mode)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int col = col0 + 2 * i;
      t[i].x = fmaf(col < mod_lim ? __ldg(mod_cols + col) : 0.0f, kLog2e, t[i].x);
      t[i].y = fmaf(col + 1 < mod_lim ? __ldg(mod_cols + col + 1) : 0.0f, kLog2e, t[i].y);
    }
  }
  float2 pv[8];
  if constexpr (kAccurate) {
#pragma unroll
    for (int i = 0; i < 8; ++i) pv[i] = sigmoid2_accurate_from_log2(t[i]);
  } else {
    if (!kMask && warp_all_negative(t)) {
#pragma unroll
      for (int i = 0; i < 8; ++i) pv[i] = sigmoid2_from_shifted_log2_deep<kBF16>(t[i]);
    } else {
      bool all_neg = false;
      if constexpr (!kMask) {
#pragma unroll
        for (int i = 0; i < 8; ++i) t[i] = __fadd2_rn(t[i], make_float2(-kDeepShift, -kDeepShift));
        all_neg = warp_all_negative(t);
      }
      if (all_neg) {
#pragma unroll
        for (int i = 0; i < 8; ++i) pv[i] = sigmoid2_from_log2_neg<kBF16>(t[i]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) pv[i] = sigmoid2_from_log2<kBF16>(t[i]);
      }
    }
  }
  uint32_t pk_p[8], pk_ds[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float2 pp = pv[i];
    if constexpr (kMask) {
      const int col = col0 + 2 * i;
      pp.x = (col >= lo && col < hi) ? pp.x : 0.0f;
      pp.y = (col + 1 >= lo && col + 1 < hi) ? pp.y : 0.0f;
    }
    const float2 w = __ffma2_rn(make_float2(-pp.x, -pp.y), pp, pp);  // P - P^2
    float2 d = __fmul2_rn(w, make_float2(__uint_as_float(rd[2 * i]), __uint_as_float(rd[2 * i + 1])));
    if constexpr (kMask) {
      d.x = (pp.x != 0.0f) ? d.x : 0.0f;  // masked elements have P exactly 0; keeps NaN/Inf padding out
      d.y = (pp.y != 0.0f) ? d.y : 0.0f;
    }
    if constexpr (kStoreP) pk_p[i] = pack2<kBF16>(pp.x, pp.y);
    pk_ds[i] = pack2<kBF16>(d.x, d.y);
  }
  if constexpr (kStoreP) tmem_st(s_addr, pk_p);
  tmem_st(dp_addr, pk_ds);
}

template <int D, bool kBF16, bool kDKV, bool kAccurate>
__global__ void __launch_bounds__(kBsThreads, 1)
sigattn_bwd_stream_kernel(const __grid_constant__ CUtensorMap r1_map, const __grid_constant__ CUtensorMap r2_map,
                          const __grid_constant__ CUtensorMap c1_map, const __grid_constant__ CUtensorMap c2_map,
                          const BwdStreamParams p) {
  using L = BsSmem<D, kDKV>;
  constexpr int kStages = L::kStages;
  constexpr int kSlots = L::kSlots;
  constexpr int kRBufs = L::kRBufs;
  constexpr int kTileBytes = L::kTileBytes;
  constexpr uint32_t kTmemCols = 512;
  // slot i: S at 128 i, dP at 128 i + 64; then out2 (dV) and out1 (dK / dQ)
  constexpr uint32_t kColOut2 = 128 * kSlots;
  constexpr uint32_t kColOut1 = kColOut2 + (kDKV ? D : 0);
  static_assert(kColOut1 + D <= kTmemCols, "TMEM budget");
  constexpr int kSiteBase = kDKV ? 0x40000 : 0x50000;
  constexpr int kItemReaders = kBsComputeWarps + 2;

  extern __shared__ uint8_t smem_dyn[];
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
  const uint32_t bars = smem_base + L::kBarOff;
  auto bar = [&](int slot) -> uint32_t { return bars + 8u * slot; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 4);
  volatile int* item_ring = reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 8);  // [2]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // a kernel of this library already gave up on a wait: do not pile more work on a sick device
  if (*reinterpret_cast<volatile int*>(&g_status_word) != 0) return;

  // ---------------------------------------------------------------- setup
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(L::kRFull + i), 1);
      mbar_init(bar(L::kREmpty + i), 1);
      mbar_init(bar(L::kItemFull + i), 1);
      mbar_init(bar(L::kItemEmpty + i), kItemReaders);
    }
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar(L::kCFull + i), 1);
      mbar_init(bar(L::kCEmpty + i), 2);  // both issuers read the streamed tiles
      mbar_init(bar(L::kCFix + i), 1);
    }
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(bar(L::kInFull + i), 1);
      mbar_init(bar(L::kOutReady + i), kBsGroupWarps);
      mbar_init(bar(L::kSlotFree + i), 1);
    }
    mbar_init(bar(L::kAccFull), 1);
    mbar_init(bar(L::kAccEmpty), kBsComputeWarps);
    fence_mbar_init();
  }
  if (warp == kBsProducerWarp && lane == 0) {
    tma_prefetch_desc(&r1_map);
    tma_prefetch_desc(&r2_map);
    tma_prefetch_desc(&c1_map);
    tma_prefetch_desc(&c2_map);
  }
  if (warp == kBsIssuerIn) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  auto read_item = [&](int k) -> int {
    const int slot = k & 1;
    if (!mbar_wait_warp(bar(L::kItemFull + slot), (uint32_t)(k >> 1) & 1u, abort_flag, kSiteBase + 30)) return -1;
    const int item = item_ring[slot];
    __syncwarp();
    if (lane == 0) mbar_arrive(bar(L::kItemEmpty + slot));
    return item;
  };

  if (warp == kBsProducerWarp) {
    // ============================================================ item scheduler + TMA producer
    // Rows of the streamed tiles beyond the valid length may hold anything (NaN included).  Masked
    // probabilities are exactly zero, but 0 * NaN is NaN inside an MMA, and the streamed rows are what
    // out1 / out2 are contracted over: they are cleared in shared memory.
    auto zero_rows = [&](uint8_t* tile, int first_bad) {
      const int n_bad = 128 - first_bad;
      for (int i = lane; i < n_bad * 8 * (D / 64); i += 32) {
        const int c = i / (n_bad * 8);
        const int rem = i % (n_bad * 8);
        *reinterpret_cast<uint4*>(tile + c * 16384 + (first_bad + rem / 8) * 128 + (rem % 8) * 16) =
            make_uint4(0, 0, 0, 0);
      }
    };
    int tile = 0;  // streamed tile pairs loaded so far (all items)
    int act = 0;   // items with work so far
    bool ok = true;
    for (int k = 0; ok; ++k) {
      const int slot = k & 1;
      ok = mbar_wait_warp(bar(L::kItemEmpty + slot), ((uint32_t)(k >> 1) & 1u) ^ 1u, abort_flag, kSiteBase + 31);
      if (!ok) break;
      int item = blockIdx.x;  // the first item needs no ticket
      if (lane == 0) {
        if (k > 0) {
          const unsigned int tk = atomicAdd(p.ticket, 1u) + gridDim.x;
          item = tk < (unsigned int)p.n_items ? (int)tk : -1;
        }
        item_ring[slot] = item;
        mbar_arrive(bar(L::kItemFull + slot));
      }
      item = __shfl_sync(0xffffffffu, item, 0);
      if (item < 0) break;
      const BsItem it = bs_decode_item<kDKV>(p, item);
      if (it.n_jobs == 0) continue;

      // stationary tiles into buffer rb, once the products of the item that used it last have read it
      const int rb = act % kRBufs;
      const uint32_t rph = (uint32_t)(act / kRBufs) & 1u;
      ok = mbar_wait_warp(bar(L::kREmpty + rb), rph ^ 1u, abort_flag, kSiteBase + 32);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(bar(L::kRFull + rb), 2 * kTileBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_4d(smem_base + L::kR1Off + rb * kTileBytes + c * 16384, &r1_map, bar(L::kRFull + rb), c * 64, it.h,
                      it.tr0 + it.r0, it.bc);
          tma_load_4d(smem_base + L::kR2Off + rb * kTileBytes + c * 16384, &r2_map, bar(L::kRFull + rb), c * 64, it.h,
                      it.tr0 + it.r0, it.bc);
        }
      }
      const int j_begin = it.hj_begin >> 1, j_end = (it.hj_end + 1) >> 1;
      int st = tile % kStages;
      uint32_t ph = (uint32_t)(tile / kStages) & 1u;
      for (int j = j_begin; j < j_end && ok; ++j) {
        ok = mbar_wait_warp(bar(L::kCEmpty + st), ph ^ 1u, abort_flag, kSiteBase + 1);
        if (!ok) break;
        if (lane == 0) {
          mbar_expect_tx(bar(L::kCFull + st), 2 * kTileBytes);
#pragma unroll
          for (int c = 0; c < D / 64; ++c) {
            tma_load_4d(smem_base + L::kC1Off + st * kTileBytes + c * 16384, &c1_map, bar(L::kCFull + st), c * 64, it.h,
                        it.tc0 + j * kBsTile, it.bc);
            tma_load_4d(smem_base + L::kC2Off + st * kTileBytes + c * 16384, &c2_map, bar(L::kCFull + st), c * 64, it.h,
                        it.tc0 + j * kBsTile, it.bc);
          }
        }
        if (j * kBsTile + kBsTile > it.Lc) {
          ok = mbar_wait_warp(bar(L::kCFull + st), ph, abort_flag, kSiteBase + 13);
          if (!ok) break;
          zero_rows(smem_gen + L::kC1Off + st * kTileBytes, it.Lc - j * kBsTile);
          zero_rows(smem_gen + L::kC2Off + st * kTileBytes, it.Lc - j * kBsTile);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(L::kCFix + st));
        }
        if (++st == kStages) { st = 0; ph ^= 1u; }
      }
      tile += j_end - j_begin;
      ++act;
    }
  } else if (warp == kBsIssuerIn) {
    // ============================================================ issuer of S = R1 C1^T and dP = R2 C2^T
    const bool leader = elect_one();
    constexpr uint32_t idesc_in = make_idesc(128, kBsJobN, kBF16, false, false);
    constexpr uint32_t kStageStep = kTileBytes >> 4;
    constexpr uint32_t kHalfStep = (kBsJobN * 128) >> 4;
    // operands with rows = M / N and the 64 contiguous elements = contraction
    const uint64_t r1_d = smem_desc_sw128(smem_base + L::kR1Off, 16, 1024);
    const uint32_t r1_lo = (uint32_t)r1_d, hi = (uint32_t)(r1_d >> 32);
    const uint32_t r2_lo = (uint32_t)smem_desc_sw128(smem_base + L::kR2Off, 16, 1024);
    const uint32_t c1_lo = (uint32_t)smem_desc_sw128(smem_base + L::kC1Off, 16, 1024);
    const uint32_t c2_lo = (uint32_t)smem_desc_sw128(smem_base + L::kC2Off, 16, 1024);
    auto issue = [&](uint32_t dcol, uint32_t a_lo, uint32_t b_lo) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t off = (uint32_t)(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
        mma_ss(leader, tmem + dcol, make_desc(a_lo + off, hi), make_desc(b_lo + off, hi), idesc_in, kk > 0);
      }
    };
    int st = 0, slot = 0, total = 0, act = 0;
    uint32_t ph = 0u, sph = 0u;
    uint32_t fix_par = 0u;  // bit st: parity of stage st's "rows cleared" barrier
    bool ok = true;
    for (int k = 0; ok; ++k) {
      const int item = read_item(k);
      if (item < 0) break;
      const BsItem it = bs_decode_item<kDKV>(p, item);
      if (it.n_jobs == 0) continue;
      const int rb = act % kRBufs;
      ok = mbar_wait_warp(bar(L::kRFull + rb), (uint32_t)(act / kRBufs) & 1u, abort_flag, kSiteBase + 3);
      const uint32_t r_off = (uint32_t)rb * kStageStep;
      for (int hj = it.hj_begin; hj < it.hj_end && ok; ++hj) {
        const bool fresh = hj == it.hj_begin || (hj & 1) == 0;
        const bool last_of_tile = hj + 1 == it.hj_end || (hj & 1) == 1;
        if (fresh) {
          ok = mbar_wait_warp(bar(L::kCFull + st), ph, abort_flag, kSiteBase + 4);
          if ((hj >> 1) * kBsTile + kBsTile > it.Lc) {
            ok = ok && mbar_wait_warp(bar(L::kCFix + st), (fix_par >> st) & 1u, abort_flag, kSiteBase + 14);
            fix_par ^= 1u << st;
          }
        }
        // the slot still holds P / dS of the job kSlots earlier until its out products are complete
        if (total >= kSlots) ok = ok && mbar_wait_warp(bar(L::kSlotFree + slot), sph ^ 1u, abort_flag, kSiteBase + 5);
        else ++total;
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t c_off = (uint32_t)st * kStageStep + (uint32_t)(hj & 1) * kHalfStep;
        issue(128u * (uint32_t)slot, r1_lo + r_off, c1_lo + c_off);
        issue(128u * (uint32_t)slot + 64u, r2_lo + r_off, c2_lo + c_off);
        mma_commit(leader, bar(L::kInFull + slot));
        if (last_of_tile) {
          mma_commit(leader, bar(L::kCEmpty + st));
          if (++st == kStages) { st = 0; ph ^= 1u; }
        }
        if (++slot == kSlots) { slot = 0; sph ^= 1u; }
      }
      if (!ok) break;
      mma_commit(leader, bar(L::kREmpty + rb));  // the stationary tiles may be overwritten once these products are complete
      ++act;
    }
  } else if (warp == kBsIssuerOut) {
    // ============================================================ issuer of out1 += dS C1 and out2 += P C2
    const bool leader = elect_one();
    constexpr uint32_t idesc_out = make_idesc(128, D, kBF16, false, true);  // A in TMEM, B rows = contraction
    constexpr uint32_t kStageStep = kTileBytes >> 4;
    constexpr uint32_t kHalfStep = (kBsJobN * 128) >> 4;
    // operands whose rows are the contraction index; the next 64-column block lies 16 KB further
    const uint64_t c1_d = smem_desc_sw128(smem_base + L::kC1Off, 16384, 1024);
    const uint32_t c1_lo = (uint32_t)c1_d, hi = (uint32_t)(c1_d >> 32);
    const uint32_t c2_lo = (uint32_t)smem_desc_sw128(smem_base + L::kC2Off, 16384, 1024);
    // acc[row, d] (+)= A[row, col] (16-bit, TMEM) . B[col, d]; the 16 columns of k-step kk sit packed in
    // TMEM columns 16 kk + [0, 8) of the source
    auto issue_acc = [&](uint32_t dcol, uint32_t acol, uint32_t b_lo, uint32_t acc0) {
#pragma unroll
      for (int kk = 0; kk < kBsJobN / 16; ++kk)
        mma_ts(leader, tmem + dcol, tmem + acol + 16 * kk, make_desc(b_lo + kk * (2048 >> 4), hi), idesc_out,
               kk > 0 ? 1u : acc0);
    };
    int st = 0, slot = 0, act = 0;
    uint32_t ph = 0u, sph = 0u;
    bool ok = true;
    for (int k = 0; ok; ++k) {
      const int item = read_item(k);
      if (item < 0) break;
      const BsItem it = bs_decode_item<kDKV>(p, item);
      if (it.n_jobs == 0) continue;
      // the accumulators still hold the previous item's results until the compute warps have read them
      if (act > 0) ok = mbar_wait_warp(bar(L::kAccEmpty), (uint32_t)(act - 1) & 1u, abort_flag, kSiteBase + 33);
      for (int hj = it.hj_begin; hj < it.hj_end && ok; ++hj) {
        const bool last_of_tile = hj + 1 == it.hj_end || (hj & 1) == 1;
        const uint32_t acc0 = hj > it.hj_begin ? 1u : 0u;
        ok = mbar_wait_warp(bar(L::kOutReady + slot), sph, abort_flag, kSiteBase + 8);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t c_off = (uint32_t)st * kStageStep + (uint32_t)(hj & 1) * kHalfStep;
        if constexpr (kDKV) issue_acc(kColOut2, 128u * (uint32_t)slot, c2_lo + c_off, acc0);
        issue_acc(kColOut1, 128u * (uint32_t)slot + 64u, c1_lo + c_off, acc0);
        mma_commit(leader, bar(L::kSlotFree + slot));
        if (last_of_tile) {
          mma_commit(leader, bar(L::kCEmpty + st));
          if (++st == kStages) { st = 0; ph ^= 1u; }
        }
        if (++slot == kSlots) { slot = 0; sph ^= 1u; }
      }
      if (!ok) break;
      mma_commit(leader, bar(L::kAccFull));
      ++act;
    }
    (void)ph;
  } else if (warp < kBsComputeWarps) {
    // ============================================================ compute warps
    const int group = warp >> 3;
    const int cg = (warp >> 2) & 1;                       // which 32 of the job's 64 columns
    const int quarter = warp & 3;
    const int lane_row = quarter * 32 + lane;             // row within the stationary tile == TMEM lane
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    const float c1 = p.scale * kLog2e;
    int slot = 0, act = 0;
    uint32_t sph = 0u, turn = 0u;
    bool ok = true;

    for (int k = 0; ok; ++k) {
      const int islot = k & 1;
      ok = mbar_wait_warp(bar(L::kItemFull + islot), (uint32_t)(k >> 1) & 1u, abort_flag, kSiteBase + 30);
      if (!ok) break;
      const int item = item_ring[islot];
      if (item < 0) break;
      const BsItem it = bs_decode_item<kDKV>(p, item);
      const int row = it.r0 + lane_row;  // index within the sequence
      if (it.n_jobs > 0) {
        float c0 = item_bias(p.bias, p.bias_scalar, it.b, kDKV ? it.Lr : it.Lc);
        const float* mod_cols = nullptr;
        if (p.score_mod) {
          const float* mod = p.score_mod + (p.cu_r ? (int64_t)it.tk0 : (int64_t)it.b * p.Tk);
          if (kDKV) { if (row < (p.cu_r ? it.Lr : p.Tr)) c0 += mod[row]; }
          else mod_cols = mod;
        }
        c0 *= kLog2e;
        const int mod_lim = p.cu_r ? it.Lc : p.Tc;
        // valid columns for this lane: [lo, hi)
        int lo, hi;
        if (kDKV) { lo = p.causal ? row : 0; hi = it.Lc; }
        else      { lo = 0; hi = p.causal ? min(it.Lc, row + 1) : it.Lc; }
        for (int hj = it.hj_begin; hj < it.hj_end; ++hj) {
          if (turn == (uint32_t)group) {
            ok = mbar_wait_warp(bar(L::kInFull + slot), sph, abort_flag, kSiteBase + 10 + group);
            if (!ok) break;
            tc_fence_after_sync();
            const int col0 = kBsJobN * hj + 32 * cg;
            const uint32_t s_addr = lane_addr + 128u * (uint32_t)slot + 32u * (uint32_t)cg;
            const uint32_t dp_addr = s_addr + 64u;
            // warp-uniform: does any lane of the tile need the element predicate for these 32 columns?
            bool need_mask = col0 + 32 > it.Lc;
            if (p.causal) need_mask = need_mask || (kDKV ? (col0 < it.r0 + kBsTile - 1) : (col0 + 32 > it.r0 + 1));
            uint32_t rs[2][16], rd[2][16];
            tmem_ld(s_addr, rs[0]);
            tmem_ld(dp_addr, rd[0]);
            tmem_ld(s_addr + 16, rs[1]);
            tmem_ld(dp_addr + 16, rd[1]);
            tmem_ld_wait_for(rs[0]);
            tmem_ld_wait_for(rd[0]);
            tmem_ld_wait_for(rs[1]);
            tmem_ld_wait_for(rd[1]);
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              if (need_mask)
                bs_unit16<kBF16, kDKV, true, kAccurate>(s_addr + 16 * u, dp_addr + 16 * u, rs[u], rd[u], c1, c0, col0 + 16 * u,
                                                        lo, hi, mod_cols, mod_lim);
              else
                bs_unit16<kBF16, kDKV, false, kAccurate>(s_addr + 16 * u, dp_addr + 16 * u, rs[u], rd[u], c1, c0, col0 + 16 * u,
                                                         lo, hi, mod_cols, mod_lim);
            }
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(L::kOutReady + slot));
          }
          if (++slot == kSlots) { slot = 0; sph ^= 1u; }
          turn ^= 1u;
        }
        if (!ok) break;
      }

      // ------------------------------------------------------------ epilogue of the item
      // dK/dV mode: column groups 0,1 store out2 (dV), groups 2,3 out1 (dK), each half of the head
      // dimension; dQ mode: every group a quarter of out1.
      const int cq = warp >> 2;
      const bool is_out1 = !kDKV || cq >= 2;
      constexpr int kCols = kDKV ? D / 2 : D / 4;  // output columns per thread
      const int col_first = kDKV ? (cq & 1) * kCols : cq * kCols;
      uint8_t* obase = reinterpret_cast<uint8_t*>(is_out1 ? p.out1 : p.out2);
      const int64_t sb = is_out1 ? p.o1_sb : p.o2_sb, stt = is_out1 ? p.o1_st : p.o2_st, sh = is_out1 ? p.o1_sh : p.o2_sh;
      uint8_t* out_row = obase + 2 * ((int64_t)it.bc * sb + (int64_t)it.h * sh + (int64_t)(it.tr0 + row) * stt) + 2 * col_first;
      if (it.n_jobs == 0) {
        // nothing on the streamed side sees this tile: its gradients are zero
        if (row < it.row_lim) {
#pragma unroll
          for (int c = 0; c < kCols / 8; ++c) *reinterpret_cast<uint4*>(out_row + 16 * c) = make_uint4(0, 0, 0, 0);
        }
      } else {
        ok = mbar_wait_warp(bar(L::kAccFull), (uint32_t)act & 1u, abort_flag, kSiteBase + 15);
        if (!ok) break;
        ++act;
        tc_fence_after_sync();
        const uint32_t acc_addr = lane_addr + (is_out1 ? kColOut1 : kColOut2) + col_first;
        const float mul = is_out1 ? p.scale : 1.0f;
        const bool live = row < it.Lr;
        uint4 w[kCols / 8];
#pragma unroll
        for (int c = 0; c < kCols / 16; ++c) {
          uint32_t r[16];
          tmem_ld(acc_addr + 16 * c, r);
          tmem_ld_wait_for(r);
#pragma unroll
          for (int q4 = 0; q4 < 2; ++q4) {
            uint4 x;
            x.x = pack2<kBF16>(mul * __uint_as_float(r[8 * q4 + 0]), mul * __uint_as_float(r[8 * q4 + 1]));
            x.y = pack2<kBF16>(mul * __uint_as_float(r[8 * q4 + 2]), mul * __uint_as_float(r[8 * q4 + 3]));
            x.z = pack2<kBF16>(mul * __uint_as_float(r[8 * q4 + 4]), mul * __uint_as_float(r[8 * q4 + 5]));
            x.w = pack2<kBF16>(mul * __uint_as_float(r[8 * q4 + 6]), mul * __uint_as_float(r[8 * q4 + 7]));
            w[2 * c + q4] = live ? x : make_uint4(0, 0, 0, 0);
          }
        }
        // the accumulators are in registers: the next item's first out products may overwrite them
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(L::kAccEmpty));
        if (row < it.row_lim) {
#pragma unroll
          for (int c = 0; c < kCols / 8; ++c) *reinterpret_cast<uint4*>(out_row + 16 * c) = w[c];
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(L::kItemEmpty + islot));
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kBsIssuerIn) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
  if (threadIdx.x == 0) {
    // the last CTA to finish leaves both counters at zero for the next launch that uses them
    __threadfence();
    const unsigned int done = atomicAdd(p.ticket + 1, 1u);
    if (done == gridDim.x - 1) {
      p.ticket[0] = 0u;
      p.ticket[1] = 0u;
      __threadfence();
    }
  }
}

}  // namespace sigattn
