// Backward kernel.  A work item is one (batch, head, 128-key tile): its K_j and V_j stay in shared
// memory, dK_j and dV_j in TMEM, and the query tiles Q_i, dO_i are streamed past them.  The kernel
// is persistent: one CTA per SM takes items from a ticket counter until none are left, so that
// the loads and first products of the next item overlap the dK/dV epilogue of the current one and
// uneven items (causal, ragged lengths) balance themselves.
//
// Takes over the work of the reference's _bwd_dense_dq_kernel / _bwd_dense_dkdv_kernel
// (src/triton_sigmoid/sigmoid_triton_dense.py:162-467) and the padded pair
// (src/triton_sigmoid/sigmoid_triton_padded.py:179-509).  The reference recomputes S and dP
// in both of its kernels (7 GEMMs per tile pair); here each tile pair costs 5:
//
//   S^T  = K_j Q_i^T            (smem x smem -> TMEM, fp32)   [key rows on TMEM lanes]
//   dP^T = V_j dO_i^T           (smem x smem -> TMEM, fp32)
//   P^T  = sigmoid(scale S^T + bias), dS^T = P^T (1 - P^T) dP^T        (registers)
//   dV_j += P^T  dO_i           (TMEM x smem -> TMEM)
//   dK_j += dS^T Q_i            (TMEM x smem -> TMEM)
//   dQ_i  = dS K_j              (smem x smem -> TMEM), then added into an fp32 accumulator in
//                                global memory.  The L2 performs such reductions at full speed
//                                only when a request covers consecutive addresses, and a warp
//                                that reads dQ with query rows on the TMEM lanes would scatter
//                                32 lanes over 32 rows.  So:
//                                D = 128: the transposed product dQ^T = K^T dS^T is computed
//                                  instead; the head dimension lies on the lanes and one
//                                  red.global.add.f32 per query covers a full 128-byte line;
//                                D = 64: the transposed product would have M = 64 and idle half of
//                                  the tensor core and half of the lanes, so dQ is kept as it is and
//                                  each warp takes full 128-byte half rows of every second query row,
//                                  regrouped through a private shared-memory patch so that eight
//                                  lanes cover a line, and adds them with red.global.add.v4.f32
//                                  (the reduction traffic, not the math, is what bounds this case).
//
// Warp roles (20 warps; 28 at D = 64):
//   warps 0-15  compute: warp w owns TMEM lanes (key rows) 32 (w & 3) .. +31 and the query
//               columns 32 (w >> 2) .. +31 of every tile; at D = 128 the same warps drain dQ
//   warp  16    item scheduler + TMA producer (also clears padded rows of tiles that straddle a valid length)
//   warp  17    tcgen05 issuer A: S^T and dP^T; owns the TMEM allocation
//   warp  18    tcgen05 issuer B: dV, dK, dQ
//   warp  19    idle
//   warps 20-27 D = 64 only: dQ drain.  The reductions into the fp32 accumulator are slow to issue (the
//               L2 serves a warp's reductions one 128-byte line at a time), and while the compute warps
//               issued them themselves (29 % of their time, measured) the MUFU unit and the tensor pipe
//               stood idle and the next tile's scores, which reuse the dQ columns, were late.  Eight
//               warps that do nothing else take dQ out of TMEM as soon as it is complete (freeing the
//               columns at once) and feed the reductions while the compute warps are two phases ahead.
//               They also take the epilogue (dK_j, dV_j) of short items, see kDrainEpilogueMaxTiles.
//               Registers are re-balanced with setmaxnreg (compute 80, role warps 72, drain warps 56 per thread);
//               to fit, the compute warps do not keep P in registers between their two phases but read its
//               16-bit copy back from TMEM.
//               (No room for this at D = 128: the drain needs its whole tile in registers or shared
//               memory before it can release the columns, and neither has any left there.)
// Two issuing warps, because one warp's instruction stream (waits, 32 MMAs, commits per tile
// pair) is a serial chain that otherwise bounds the kernel.  Everything the two exchange goes
// through mbarriers: "S columns free" after dV, "dP columns free" after dK.
// dQ = scale * accumulator is rounded to the 16-bit type by sigattn_dq_convert_kernel.
#pragma once

#include "ptx.cuh"
#include "sigmoid_math.cuh"

namespace sigattn {

struct BwdParams {
  float* dq_acc;  // [B, Tq, H, D] fp32, zero-filled before the launch
  void* dk;
  void* dv;
  int64_t dk_sb, dk_st, dk_sh;
  int64_t dv_sb, dv_st, dv_sh;
  const int* lens_q;
  const int* lens_k;
  // Packed (variable-length) layout: sequence b occupies rows cu_q[b] .. cu_q[b+1]-1 of a (total, H, D)
  // tensor (likewise cu_k for keys / values); Tq, Tk are then upper bounds of the lengths and dq_acc is
  // [total queries, H, D].  nullptr = (B, T, H, D).
  const int* cu_q;
  const int* cu_k;
  const float* bias;
  const float* score_mod;
  float scale;
  float bias_scalar;
  int B, H, Tq, Tk;
  int causal;
  int n_kvblk;  // ceil(Tk / 128)
  int n_items;  // B * H * n_kvblk
  int group;    // (batch, head) pairs per scheduling group, >= 1 (see bwd_decode_item)
  // two counters, zero between launches: [0] items handed out beyond the first per CTA,
  // [1] CTAs that have finished (the last one clears both)
  unsigned int* ticket;
};

constexpr int kBwdComputeWarps = 16;
constexpr int kBwdProducerWarp = 16;
constexpr int kBwdIssuerA = 17;
constexpr int kBwdIssuerB = 18;
constexpr int kBwdDrainWarps = 8;
// D = 64: the drain warps also take the epilogue (dK_j, dV_j out of TMEM and to global memory) of items with at most
// this many query tiles, so that the compute warps go straight on to the next item; for longer items, whose
// epilogue is a small share, the compute warps do it themselves (the drain warps, busy with it, would fall
// behind with the next item's dQ tiles: measured -1.5 % at 32 tiles per item, +7 % at 4).
constexpr int kDrainEpilogueMaxTiles = 8;    // D = 64 only
constexpr int kBwdFirstDrainWarp = 20;
template <int D> constexpr int kBwdThreads = (D == 64) ? (kBwdFirstDrainWarp + kBwdDrainWarps) * 32 : 20 * 32;
constexpr int kBwdTileKV = 128;
constexpr int kBwdTileQ = 128;

template <int D>
struct BwdSmem {
  static constexpr int kStages = 2;
  static constexpr int kTileBytes = 128 * D * 2;
  // K_j / V_j buffers: two at D = 64 (the next item's are loaded while this item still computes), one at
  // D = 128 (no room for more)
  static constexpr int kKvBufs = (D == 64) ? 2 : 1;
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kKOff + kKvBufs * kTileBytes;
  static constexpr int kQOff = kVOff + kKvBufs * kTileBytes;
  static constexpr int kDoOff = kQOff + kStages * kTileBytes;
  static constexpr int kDsOff = kDoOff + kStages * kTileBytes;
  static constexpr int kDsBytes = 128 * 128 * 2;
  // D = 64 only: a private patch of 32 rows x 128 bytes per drain warp, used to regroup dQ rows so
  // that eight adjacent lanes add the 128 bytes of one row (16 bytes of padding per row keep the
  // 16-byte accesses of different rows off each other's banks)
  static constexpr int kDqPatchRow = 128 + 16;
  static constexpr int kDqPatchOff = kDsOff + kDsBytes;
  static constexpr int kDqPatchBytes = (D == 64) ? 32 * kDqPatchRow : 0;
  static constexpr int kBarOff = kDqPatchOff + kBwdDrainWarps * kDqPatchBytes;
  static constexpr int kKvFull = 0;                   // [2] per K/V buffer
  static constexpr int kQFull = 2;                    // [2]
  static constexpr int kQEmpty = kQFull + kStages;    // [2]  both issuers release a stage
  static constexpr int kDoFull = kQEmpty + kStages;   // [2]
  static constexpr int kDoEmpty = kDoFull + kStages;  // [2]
  static constexpr int kSFull = kDoEmpty + kStages;   // [2] S^T written (per S buffer)
  static constexpr int kDpFull = kSFull + 2;          // dP^T written
  static constexpr int kPReady = kDpFull + 1;         // [2] P^T in TMEM (16 warps; per S buffer)
  static constexpr int kDsReady = kPReady + 2;        // dS^T in TMEM and shared memory (16 warps)
  static constexpr int kSFree = kDsReady + 1;         // dV has consumed P^T: S columns reusable
  static constexpr int kDpFree = kSFree + 1;          // dK has consumed dS^T: dP columns reusable
  static constexpr int kDqFull = kDpFree + 1;         // [2] dQ tile complete in TMEM
  static constexpr int kDqEmpty = kDqFull + 2;        // [2] dQ tile read out (16 warps)
  static constexpr int kDkvFull = kDqEmpty + 2;       // every MMA of the CTA complete
  static constexpr int kKvFix = kDkvFull + 1;         // [2] per K/V buffer: padded rows of K_j zeroed
  static constexpr int kQdoFix = kKvFix + 2;          // [2] per stage: padded rows of the last Q_i / dO_i zeroed
  static constexpr int kKvEmpty = kQdoFix + 2;        // [2] per K/V buffer, both issuers: every product that reads it is complete
  static constexpr int kDkvEmpty = kKvEmpty + 2;      // [2] dK_j, dV_j read out of TMEM: [0] by the 16 compute warps, [1] by the 8 drain warps (short items at D = 64)
  static constexpr int kItemFull = kDkvEmpty + 2;     // [2] item index published
  static constexpr int kItemEmpty = kItemFull + 2;    // [2] item index read by every consumer warp
  static constexpr int kNumBars = kItemEmpty + 2;
  static constexpr int kMiscOff = kBarOff + 8 * kNumBars;  // tmem base (u32), abort flag (int), 2 x item record (16 int each)
  static constexpr int kTotal = kMiscOff + 16 + 2 * 64;
  static constexpr int kDynBytes = kTotal + 1024;
};

// Phase A of one tile for one thread: 32 scores of its key row -> probabilities (kept in pv[]
// for phase B) and their 16-bit packing written over the first 16 of the 32 columns read.
// q0 = query index of the first column; valid queries for this key row are [q_lo, q_hi).
template <bool kBF16, bool kMask, bool kAccurate>
__device__ __forceinline__ void bwd_phase_a(uint32_t s_addr, float c1, float c0, int q0, int q_lo, int q_hi,
                                            float (&pv)[32]) {
  uint32_t r[32];
  tmem_ld32_sync(s_addr, r);
  uint32_t pk[16];
  float2 t[16];
  // unmasked tiles work on logits shifted up by kDeepShift (see sigmoid2_from_shifted_log2_deep)
  const float c0s = (kMask || kAccurate) ? c0 : c0 + kDeepShift;
#pragma unroll
  for (int i = 0; i < 16; ++i)
    t[i] = __ffma2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), make_float2(c1, c1),
                      make_float2(c0s, c0s));
  if constexpr (kAccurate) {
    // exponential and reciprocal both on the special-function unit (see sigmoid2_accurate_from_log2)
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float2 pe = sigmoid2_accurate_from_log2(t[i]);
      if constexpr (kMask) {
        const int q = q0 + 2 * i;
        pe.x = (q >= q_lo && q < q_hi) ? pe.x : 0.0f;
        pe.y = (q + 1 >= q_lo && q + 1 < q_hi) ? pe.y : 0.0f;
      }
      pv[2 * i] = pe.x;
      pv[2 * i + 1] = pe.y;
      pk[i] = pack2<kBF16>(pe.x, pe.y);
    }
  } else
  // all logits far below zero (the usual case under the default bias): short series, no compare / select per element
  if (!kMask && warp_all_negative(t)) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float2 pe = sigmoid2_from_shifted_log2_deep<kBF16>(t[i]);
      pv[2 * i] = pe.x;
      pv[2 * i + 1] = pe.y;
      pk[i] = pack2<kBF16>(pe.x, pe.y);
    }
  } else {
    bool all_neg = false;
    if constexpr (!kMask) {
#pragma unroll
      for (int i = 0; i < 16; ++i) t[i] = __fadd2_rn(t[i], make_float2(-kDeepShift, -kDeepShift));
      all_neg = warp_all_negative(t);  // negative but not far below zero: full polynomial, still no select
    }
    if (all_neg) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float2 pe = sigmoid2_from_log2_neg<kBF16>(t[i]);
        pv[2 * i] = pe.x;
        pv[2 * i + 1] = pe.y;
        pk[i] = pack2<kBF16>(pe.x, pe.y);
      }
    } else
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float2 pe = sigmoid2_from_log2<kBF16>(t[i]);
      if constexpr (kMask) {
        const int q = q0 + 2 * i;
        pe.x = (q >= q_lo && q < q_hi) ? pe.x : 0.0f;
        pe.y = (q + 1 >= q_lo && q + 1 < q_hi) ? pe.y : 0.0f;
      }
      pv[2 * i] = pe.x;
      pv[2 * i + 1] = pe.y;
      pk[i] = pack2<kBF16>(pe.x, pe.y);
    }
  }
  tmem_st16(s_addr, pk);
}

// Phase B: dS = P (1 - P) dP for the same 32 columns; 16-bit dS^T goes to TMEM (over the first
// 16 dP columns read) and to the swizzled shared-memory copy the dQ GEMM reads.
template <bool kBF16, bool kMask>
__device__ __forceinline__ void bwd_phase_b(uint32_t dp_addr, uint32_t ds_line, uint32_t chunk0, uint32_t sw,
                                            const float (&pv)[32]) {
  uint32_t r[32];
  tmem_ld32_sync(dp_addr, r);
  uint32_t pk[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float2 pp = make_float2(pv[2 * i], pv[2 * i + 1]);
    const float2 w = __ffma2_rn(make_float2(-pp.x, -pp.y), pp, pp);  // P - P^2
    float2 d = __fmul2_rn(w, make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])));
    if constexpr (kMask) {
      d.x = (pp.x != 0.0f) ? d.x : 0.0f;  // masked elements have P exactly 0; keeps NaN/Inf padding out
      d.y = (pp.y != 0.0f) ? d.y : 0.0f;
    }
    pk[i] = pack2<kBF16>(d.x, d.y);
  }
  tmem_st16(dp_addr, pk);
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    const uint32_t chunk = (chunk0 + m) ^ sw;  // 128-byte swizzle: 16-byte chunk index XOR (row & 7)
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(ds_line + chunk * 16), "r"(pk[4 * m]),
                 "r"(pk[4 * m + 1]), "r"(pk[4 * m + 2]), "r"(pk[4 * m + 3])
                 : "memory");
  }
}

// The two phases for the D = 64 kernel.  The probabilities are not kept in registers between the phases
// (32 registers per thread that the drain warps' share of the register file cannot spare) but read back
// from TMEM in the 16-bit form they were stored in for the dV product, and dS = P (1 - P) dP is formed on
// packed 16-bit pairs.
template <bool kBF16, bool kMask, bool kAccurate>
__device__ __forceinline__ void bwd_phase_a16(uint32_t s_addr, float c1, float c0, int q0, int q_lo, int q_hi) {
  uint32_t r[32];
  tmem_ld32_sync(s_addr, r);
  uint32_t pk[16];
  float2 t[16];
  const float c0s = (kMask || kAccurate) ? c0 : c0 + kDeepShift;
#pragma unroll
  for (int i = 0; i < 16; ++i)
    t[i] = __ffma2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), make_float2(c1, c1),
                      make_float2(c0s, c0s));
  if constexpr (kAccurate) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float2 pe = sigmoid2_accurate_from_log2(t[i]);
      if constexpr (kMask) {
        const int q = q0 + 2 * i;
        pe.x = (q >= q_lo && q < q_hi) ? pe.x : 0.0f;
        pe.y = (q + 1 >= q_lo && q + 1 < q_hi) ? pe.y : 0.0f;
      }
      pk[i] = pack2<kBF16>(pe.x, pe.y);
    }
  } else if (!kMask && warp_all_negative(t)) {
    // all logits far below zero (the usual case under the default bias): short series on packed pairs
#pragma unroll
    for (int i = 0; i < 16; ++i) pk[i] = sigmoid2_deep_packed<kBF16>(t[i], false);
  } else {
    bool all_neg = false;
    if constexpr (!kMask) {
#pragma unroll
      for (int i = 0; i < 16; ++i) t[i] = __fadd2_rn(t[i], make_float2(-kDeepShift, -kDeepShift));
      all_neg = warp_all_negative(t);
    }
    if (all_neg) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float2 pe = sigmoid2_from_log2_neg<kBF16>(t[i]);
        pk[i] = pack2<kBF16>(pe.x, pe.y);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float2 pe = sigmoid2_from_log2<kBF16>(t[i]);
        if constexpr (kMask) {
          const int q = q0 + 2 * i;
          pe.x = (q >= q_lo && q < q_hi) ? pe.x : 0.0f;
          pe.y = (q + 1 >= q_lo && q + 1 < q_hi) ? pe.y : 0.0f;
        }
        pk[i] = pack2<kBF16>(pe.x, pe.y);
      }
    }
  }
  tmem_st16(s_addr, pk);
}

template <bool kBF16, bool kMask>
__device__ __forceinline__ void bwd_phase_b16(uint32_t p_addr, uint32_t dp_addr, uint32_t ds_line, uint32_t chunk0,
                                              uint32_t sw) {
  uint32_t pp[16], r[32];
  tmem_ld16(p_addr, pp);
  tmem_ld32(dp_addr, r);
  tmem_ld_wait_for(pp);
  tmem_ld_wait_for(r);
  uint32_t pk[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t ph = pp[i];
    const uint32_t w = hfma2<kBF16>(ph ^ 0x80008000u, ph, ph);  // P - P^2
    uint32_t d = hmul2<kBF16>(w, pack2<kBF16>(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])));
    if constexpr (kMask) {
      // masked elements have P exactly 0: force dS to 0 there, whatever (NaN, Inf) the padding put into dP
      const uint32_t keep = ((ph & 0x00007fffu) ? 0x0000ffffu : 0u) | ((ph & 0x7fff0000u) ? 0xffff0000u : 0u);
      d &= keep;
    }
    pk[i] = d;
  }
  tmem_st16(dp_addr, pk);
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    const uint32_t chunk = (chunk0 + m) ^ sw;  // 128-byte swizzle: 16-byte chunk index XOR (row & 7)
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(ds_line + chunk * 16), "r"(pk[4 * m]),
                 "r"(pk[4 * m + 1]), "r"(pk[4 * m + 2]), "r"(pk[4 * m + 3])
                 : "memory");
  }
}

// One work item.  The producer warp decodes it once (integer divisions, length and bias loads from global
// memory) and publishes the record through shared memory; every other role reads it from there.
struct BwdItem {
  int b, h, kv0;
  int bc;               // batch coordinate of the tensor maps and strides (0 when packed)
  int tq0, tk0;         // first row of the sequence in the token dimension (0 unless packed)
  int key_lim;          // key rows below this exist in this sequence's tensors (Tk; packed: Lk)
  int64_t acc_row0;     // first row of the sequence in the dQ accumulator
  int Lq, Lk;
  int i_begin, n_q;     // first query tile that sees this key tile, number of query tiles
  bool ragged_kv;       // the key tile straddles Lk
  bool ragged_last_q;   // the last query tile straddles Lq
  float bias;           // additive bias of the item's batch element
};
// record layout in shared memory: 16 ints, [0] = item index (-1: no more work)
__device__ __forceinline__ void bwd_publish_item(volatile int* rec, int item, const BwdItem& it) {
  rec[1] = it.b; rec[2] = it.h; rec[3] = it.kv0; rec[4] = it.bc; rec[5] = it.tq0; rec[6] = it.tk0; rec[7] = it.key_lim;
  rec[8] = (int)(uint32_t)((uint64_t)it.acc_row0 & 0xffffffffull); rec[9] = (int)(uint32_t)((uint64_t)it.acc_row0 >> 32);
  rec[10] = it.Lq; rec[11] = it.Lk; rec[12] = it.i_begin; rec[13] = it.n_q;
  rec[14] = (it.ragged_kv ? 1 : 0) | (it.ragged_last_q ? 2 : 0); rec[15] = __float_as_int(it.bias);
  rec[0] = item;
}
__device__ __forceinline__ BwdItem bwd_load_item(const volatile int* rec) {
  BwdItem it;
  it.b = rec[1]; it.h = rec[2]; it.kv0 = rec[3]; it.bc = rec[4]; it.tq0 = rec[5]; it.tk0 = rec[6]; it.key_lim = rec[7];
  it.acc_row0 = (int64_t)(((uint64_t)(uint32_t)rec[9] << 32) | (uint64_t)(uint32_t)rec[8]);
  it.Lq = rec[10]; it.Lk = rec[11]; it.i_begin = rec[12]; it.n_q = rec[13];
  const int fl = rec[14];
  it.ragged_kv = (fl & 1) != 0; it.ragged_last_q = (fl & 2) != 0; it.bias = __int_as_float(rec[15]);
  return it;
}
__device__ __forceinline__ BwdItem bwd_decode_item(const BwdParams& p, int item) {
  BwdItem it;
  // Groups of `group` (batch, head) pairs: within a group every pair's key tile 0 comes first, then
  // every pair's tile 1, ... (under a causal mask the early tiles are the heavy ones, so this is a
  // longest-first order), while the Q / dO of one group still fit the L2.  group = 1: (batch, head)-major.
  const int per_group = p.group * p.n_kvblk;
  const int grp = item / per_group;
  const int r = item - grp * per_group;
  const int g_eff = min(p.group, p.B * p.H - grp * p.group);
  const int j = r / g_eff;  // key tile
  const int bh = grp * p.group + (r - j * g_eff);
  it.b = bh / p.H;
  it.h = bh - it.b * p.H;
  it.kv0 = j * kBwdTileKV;
  it.Lq = p.Tq;
  it.Lk = p.Tk;
  if (p.lens_q) it.Lq = min(max(p.lens_q[it.b], 0), p.Tq);
  if (p.lens_k) it.Lk = min(max(p.lens_k[it.b], 0), p.Tk);
  it.bc = it.b;
  it.tq0 = it.tk0 = 0;
  it.key_lim = p.Tk;
  it.acc_row0 = (int64_t)it.b * p.Tq;
  if (p.cu_q) {
    it.tq0 = p.cu_q[it.b];
    it.tk0 = p.cu_k[it.b];
    it.Lq = min(max(p.cu_q[it.b + 1] - it.tq0, 0), p.Tq);
    it.Lk = min(max(p.cu_k[it.b + 1] - it.tk0, 0), p.Tk);
    it.bc = 0;
    it.key_lim = it.Lk;
    it.acc_row0 = it.tq0;
  }
  const int i_end = (it.Lq + kBwdTileQ - 1) / kBwdTileQ;
  it.i_begin = p.causal ? j : 0;  // query tiles that can see this key tile (top-left aligned)
  it.n_q = (it.kv0 < it.Lk) ? max(i_end - it.i_begin, 0) : 0;
  it.ragged_kv = it.kv0 + kBwdTileKV > it.Lk;
  it.ragged_last_q = (it.i_begin + it.n_q) * kBwdTileQ > it.Lq;  // only the last query tile can straddle Lq
  it.bias = item_bias(p.bias, p.bias_scalar, it.b, it.Lk);
  return it;
}

template <int D, bool kBF16, bool kAccurate>
__global__ void __launch_bounds__(kBwdThreads<D>, 1)
sigattn_bwd_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                   const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap do_map,
                   const BwdParams p) {
  using L = BwdSmem<D>;
  constexpr int kTileBytes = L::kTileBytes;
  constexpr uint32_t kTmemCols = 512;
  // TMEM plan.  D = 64: two S^T buffers (tiles alternate), so that the scores of the next tile are
  // computed while this one is still being processed; dQ_i is written over the S^T buffer of its
  // own tile once dV has read P^T from it:   S0 0 | S1 128 | dP 256 | dV 384 | dK 448.
  // D = 128: no room for that: one S^T buffer, dQ^T over the dP^T columns:  S 0 | dP 128 | dV 256 | dK 384.
  // Column group c keeps its 16-bit P^T in S columns 32c + [0,16), dS^T likewise in the dP columns.
  constexpr bool kTwoS = (D == 64);
  constexpr bool kDqT = (D == 128);         // dQ^T (head dimension on lanes) instead of dQ
  constexpr uint32_t kColS = 0;
  constexpr uint32_t kColDp = kTwoS ? 256 : 128;
  constexpr uint32_t kColDv = kTwoS ? 384 : 256;
  constexpr uint32_t kColDk = kColDv + D;
  static_assert(kColDk + D <= kTmemCols, "TMEM budget");
  // Query tiles are numbered through the whole life of the CTA (g = tiles of earlier items + index
  // within the item): stages, S buffers and barrier parities simply run on from item to item.
  // index and parity of the per-S-buffer barriers for tile g
  auto sbuf = [](int g) -> int { return kTwoS ? (g & 1) : 0; };
  auto spar = [](int g) -> uint32_t { return kTwoS ? (uint32_t)(g >> 1) & 1u : (uint32_t)g & 1u; };
  // where dQ (or dQ^T) of tile g is written
  auto dq_col = [&](int g) -> uint32_t { return kTwoS ? kColS + 128u * (uint32_t)(g & 1) : kColDp; };
  constexpr int kSiteBase = 0x20000;
  constexpr bool kDrainWarps = kTwoS;  // dedicated dQ drain warps (see the file header)
  // compute warps, the two issuing warps and the drain warps read the item ring
  constexpr int kItemReaders = kBwdComputeWarps + 2 + (kDrainWarps ? kBwdDrainWarps : 0);

  extern __shared__ uint8_t smem_dyn[];
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
  const uint32_t bars = smem_base + L::kBarOff;
  auto bar = [&](int slot) -> uint32_t { return bars + 8u * slot; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 4);
  volatile int* item_ring = reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 16);  // 2 records of 16 ints

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // a kernel of this library already gave up on a wait: do not pile more work on a sick device
  if (*reinterpret_cast<volatile int*>(&g_status_word) != 0) return;

  // ---------------------------------------------------------------- setup
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(L::kKvFull + i), 1);
      mbar_init(bar(L::kKvFix + i), 1);
      mbar_init(bar(L::kQdoFix + i), 1);
      mbar_init(bar(L::kKvEmpty + i), 2);  // issuer A (S^T, dP^T) and issuer B (dQ)
    }
    for (int i = 0; i < L::kStages; ++i) {
      mbar_init(bar(L::kQFull + i), 1);
      mbar_init(bar(L::kQEmpty + i), 2);   // S^T (issuer A) and dK (issuer B) both read Q_i
      mbar_init(bar(L::kDoFull + i), 1);
      mbar_init(bar(L::kDoEmpty + i), 2);  // dP^T (issuer A) and dV (issuer B) both read dO_i
    }
    mbar_init(bar(L::kSFull + 0), 1);
    mbar_init(bar(L::kSFull + 1), 1);
    mbar_init(bar(L::kDpFull), 1);
    mbar_init(bar(L::kPReady + 0), kBwdComputeWarps);
    mbar_init(bar(L::kPReady + 1), kBwdComputeWarps);
    mbar_init(bar(L::kDsReady), kBwdComputeWarps);
    mbar_init(bar(L::kSFree), 1);
    mbar_init(bar(L::kDpFree), 1);
    mbar_init(bar(L::kDqFull + 0), 1);
    mbar_init(bar(L::kDqFull + 1), 1);
    mbar_init(bar(L::kDqEmpty + 0), kDrainWarps ? kBwdDrainWarps : kBwdComputeWarps);
    mbar_init(bar(L::kDqEmpty + 1), kDrainWarps ? kBwdDrainWarps : kBwdComputeWarps);
    mbar_init(bar(L::kDkvFull), 1);
    mbar_init(bar(L::kDkvEmpty + 0), kBwdComputeWarps);
    mbar_init(bar(L::kDkvEmpty + 1), kBwdDrainWarps);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(L::kItemFull + i), 1);
      mbar_init(bar(L::kItemEmpty + i), kItemReaders);
    }
    fence_mbar_init();
  }
  if (warp == kBwdProducerWarp && lane == 0) {
    tma_prefetch_desc(&q_map);
    tma_prefetch_desc(&k_map);
    tma_prefetch_desc(&v_map);
    tma_prefetch_desc(&do_map);
  }
  if (warp == kBwdIssuerA) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  // Consumer side of the item ring: returns the k-th item of this CTA, or -1 when there is none
  // (also on a failed wait).  Called by all 32 lanes of a reader warp.
  auto read_item = [&](int k, BwdItem& it) -> int {
    const int slot = k & 1;
    if (!mbar_wait_warp(bar(L::kItemFull + slot), (uint32_t)(k >> 1) & 1u, abort_flag, kSiteBase + 30)) return -1;
    const int item = item_ring[16 * slot];
    if (item >= 0) it = bwd_load_item(item_ring + 16 * slot);
    __syncwarp();
    if (lane == 0) mbar_arrive(bar(L::kItemEmpty + slot));
    return item;
  };

  if constexpr (kDrainWarps) {
    // 896 threads get 72 registers each at launch.  Each aligned group of four warps executes one
    // instruction; the counts add up to exactly what the CTA holds (512 x 80 + 128 x 72 + 256 x 56).
    // (The issuing warps are the ones that must not spill: their instruction stream is the critical chain.)
    if (warp < kBwdComputeWarps)         setmaxnreg_inc<80>();
    else if (warp >= kBwdFirstDrainWarp) setmaxnreg_dec<56>();
  }

  if (kDrainWarps && warp >= kBwdFirstDrainWarp) {
    // ============================================================ dQ drain (D = 64)
    // Warp d = warp - 20: lane quarter d & 3 (32 query rows), head columns [32 (d >> 2), +32) = one 128-byte
    // line of the accumulator per row.  Per tile: wait for the dQ product, move the 32 x 32 block through
    // registers into the warp's shared-memory patch, release the TMEM columns, then add the rows into the
    // accumulator with red.global.add.v4.f32, eight adjacent lanes per line.
    if constexpr (kDrainWarps) {
      const int dw = warp - kBwdFirstDrainWarp;
      const int quarter = dw & 3, half = dw >> 2;
      const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
      uint8_t* patch = smem_gen + L::kDqPatchOff + dw * L::kDqPatchBytes;
      int g = 0;
      int act = 0;  // items with work so far
      bool ok = true;
      for (int k = 0; ok; ++k) {
        BwdItem it;
        const int item = read_item(k, it);
        if (item < 0) break;
        if (it.n_q == 0) continue;
        for (int t = 0; t < it.n_q && ok; ++t) {
          const int gt = g + t;
          ok = mbar_wait_warp(bar(L::kDqFull + sbuf(gt)), spar(gt), abort_flag, kSiteBase + 14);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t addr = tmem + lane_addr + dq_col(gt) + 32u * (uint32_t)half;
          uint4* mine = reinterpret_cast<uint4*>(patch + lane * L::kDqPatchRow);
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            uint32_t r[16];
            tmem_ld(addr + 16 * u, r);
            tmem_ld_wait_for(r);
#pragma unroll
            for (int m = 0; m < 4; ++m) mine[4 * u + m] = make_uint4(r[4 * m], r[4 * m + 1], r[4 * m + 2], r[4 * m + 3]);
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(L::kDqEmpty + sbuf(gt)));  // the TMEM columns are free again
          const int q_tile = (it.i_begin + t) * kBwdTileQ + quarter * 32;
          const int slot = lane >> 3, chunk = lane & 7;  // patch row within a group of four, 16-byte chunk of the row
#pragma unroll
          for (int kq = 0; kq < 8; ++kq) {
            const int prow = 4 * kq + slot;
            const int q = q_tile + prow;
            const uint4 w = *reinterpret_cast<const uint4*>(patch + prow * L::kDqPatchRow + chunk * 16);
            if (q < it.Lq) {  // queries at or beyond Lq get no gradient
              float* dst = p.dq_acc + ((it.acc_row0 + q) * p.H + it.h) * D + 32 * half + 4 * chunk;
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(w.x)),
                           "f"(__uint_as_float(w.y)), "f"(__uint_as_float(w.z)), "f"(__uint_as_float(w.w))
                           : "memory");
            }
          }
          __syncwarp();  // the patch is rewritten at the next tile
        }
        if (!ok) break;
        g += it.n_q;

        // ---- epilogue of the item: dV_j, then dK_j, out of TMEM, rounded, through the patch (so that four
        // lanes cover a row's 64 bytes and an instruction 8 rows; a lane writing its own row would touch 32
        // lines per instruction, which the load/store unit takes one at a time) and out to global memory,
        // while the compute warps are already on the next item's first tiles.
        if (it.n_q > kDrainEpilogueMaxTiles) {
          ++act;  // the compute warps' business
          continue;
        }
        ok = mbar_wait_warp(bar(L::kDkvFull), (uint32_t)act & 1u, abort_flag, kSiteBase + 15);
        if (!ok) break;
        ++act;
        tc_fence_after_sync();
        const bool row_ok = it.kv0 + quarter * 32 + lane < it.Lk;  // padded key rows get zero gradients
#pragma unroll
        for (int which = 0; which < 2; ++which) {  // 0: dV, 1: dK
          const uint32_t acc_addr = tmem + lane_addr + (which ? kColDk : kColDv) + 32u * (uint32_t)half;
          const float mul = which ? p.scale : 1.0f;
          uint4* mine = reinterpret_cast<uint4*>(patch + lane * L::kDqPatchRow);
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            uint32_t r[16];
            tmem_ld(acc_addr + 16 * u, r);
            tmem_ld_wait_for(r);
#pragma unroll
            for (int m = 0; m < 2; ++m) {
              uint4 w;
              w.x = pack2<kBF16>(mul * __uint_as_float(r[8 * m + 0]), mul * __uint_as_float(r[8 * m + 1]));
              w.y = pack2<kBF16>(mul * __uint_as_float(r[8 * m + 2]), mul * __uint_as_float(r[8 * m + 3]));
              w.z = pack2<kBF16>(mul * __uint_as_float(r[8 * m + 4]), mul * __uint_as_float(r[8 * m + 5]));
              w.w = pack2<kBF16>(mul * __uint_as_float(r[8 * m + 6]), mul * __uint_as_float(r[8 * m + 7]));
              if (!row_ok) w = make_uint4(0, 0, 0, 0);
              mine[2 * u + m] = w;
            }
          }
          if (which == 1) {
            // both accumulators are out of TMEM: the next item's first dV / dK products may overwrite them
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(L::kDkvEmpty + 1));
          }
          __syncwarp();
          const int64_t out_st = which ? p.dk_st : p.dv_st;
          uint8_t* out = which ? reinterpret_cast<uint8_t*>(p.dk) + 2 * ((int64_t)it.bc * p.dk_sb + (int64_t)it.h * p.dk_sh + (int64_t)it.tk0 * p.dk_st)
                               : reinterpret_cast<uint8_t*>(p.dv) + 2 * ((int64_t)it.bc * p.dv_sb + (int64_t)it.h * p.dv_sh + (int64_t)it.tk0 * p.dv_st);
          out += 64 * half + 16 * (lane & 3);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r8 = 8 * i + (lane >> 2);
            const uint4 x = *reinterpret_cast<const uint4*>(patch + r8 * L::kDqPatchRow + 16 * (lane & 3));
            const int krow = it.kv0 + quarter * 32 + r8;
            if (krow < it.key_lim) *reinterpret_cast<uint4*>(out + 2 * (int64_t)krow * out_st) = x;
          }
          __syncwarp();  // the patch is rewritten by the next pass / the next item's first dQ tile
        }
      }
    }
  } else
  if (warp == kBwdProducerWarp) {
    // ============================================================ item scheduler + TMA producer
    // Rows beyond the valid lengths may hold anything (NaN included).  Masked probabilities are
    // exactly zero, but 0 * NaN is NaN inside an MMA, so the padded rows of every tile that is
    // contracted over its rows (K_j for dQ, Q_i for dK, dO_i for dV) are cleared in shared memory.
    auto zero_rows = [&](uint8_t* tile, int first_bad) {
      const int n_bad = 128 - first_bad;
      for (int i = lane; i < n_bad * 8 * (D / 64); i += 32) {
        const int c = i / (n_bad * 8);
        const int rem = i % (n_bad * 8);
        *reinterpret_cast<uint4*>(tile + c * 16384 + (first_bad + rem / 8) * 128 + (rem % 8) * 16) =
            make_uint4(0, 0, 0, 0);
      }
    };
    int g = 0;    // query tiles loaded so far (all items)
    int act = 0;  // items with work so far
    bool ok = true;
    for (int k = 0; ok; ++k) {
      const int slot = k & 1;
      ok = mbar_wait_warp(bar(L::kItemEmpty + slot), ((uint32_t)(k >> 1) & 1u) ^ 1u, abort_flag, kSiteBase + 31);
      if (!ok) break;
      int item = blockIdx.x;  // the first item needs no ticket
      if (lane == 0 && k > 0) {
        const unsigned int tk = atomicAdd(p.ticket, 1u) + gridDim.x;
        item = tk < (unsigned int)p.n_items ? (int)tk : -1;
      }
      item = __shfl_sync(0xffffffffu, item, 0);
      BwdItem it = {};
      if (item >= 0) it = bwd_decode_item(p, item);
      if (lane == 0) {
        if (item >= 0) bwd_publish_item(item_ring + 16 * slot, item, it);
        else item_ring[16 * slot] = -1;
        mbar_arrive(bar(L::kItemFull + slot));  // (release: the record is visible to whoever sees the phase)
      }
      if (item < 0) break;
      if (it.n_q == 0) continue;

      for (int t = 0; t < it.n_q && ok; ++t) {
        const int gt = g + t;
        const int st = gt & 1;
        const uint32_t ph = (uint32_t)(gt >> 1) & 1u;
        const int qrow = (it.i_begin + t) * kBwdTileQ;
        ok = mbar_wait_warp(bar(L::kQEmpty + st), ph ^ 1u, abort_flag, kSiteBase + 1);
        if (!ok) break;
        if (lane == 0) {
          mbar_expect_tx(bar(L::kQFull + st), kTileBytes);
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_4d(smem_base + L::kQOff + st * kTileBytes + c * 16384, &q_map, bar(L::kQFull + st), c * 64, it.h, it.tq0 + qrow, it.bc);
        }
        ok = mbar_wait_warp(bar(L::kDoEmpty + st), ph ^ 1u, abort_flag, kSiteBase + 2);
        if (!ok) break;
        if (lane == 0) {
          mbar_expect_tx(bar(L::kDoFull + st), kTileBytes);
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_4d(smem_base + L::kDoOff + st * kTileBytes + c * 16384, &do_map, bar(L::kDoFull + st), c * 64, it.h, it.tq0 + qrow, it.bc);
        }
        if (t == 0) {
          // K_j, V_j of this item into buffer kb, once the products of the item that used it last have
          // finished reading it (the first Q / dO tiles above are already on their way)
          const int kb = act % L::kKvBufs;
          const uint32_t kph = (uint32_t)(act / L::kKvBufs) & 1u;
          ok = mbar_wait_warp(bar(L::kKvEmpty + kb), kph ^ 1u, abort_flag, kSiteBase + 32);
          if (!ok) break;
          if (lane == 0) {
            mbar_expect_tx(bar(L::kKvFull + kb), 2 * kTileBytes);
#pragma unroll
            for (int c = 0; c < D / 64; ++c) {
              tma_load_4d(smem_base + L::kKOff + kb * kTileBytes + c * 16384, &k_map, bar(L::kKvFull + kb), c * 64, it.h, it.tk0 + it.kv0, it.bc);
              tma_load_4d(smem_base + L::kVOff + kb * kTileBytes + c * 16384, &v_map, bar(L::kKvFull + kb), c * 64, it.h, it.tk0 + it.kv0, it.bc);
            }
          }
          if (it.ragged_kv) {
            ok = mbar_wait_warp(bar(L::kKvFull + kb), kph, abort_flag, kSiteBase + 17);
            if (!ok) break;
            zero_rows(smem_gen + L::kKOff + kb * kTileBytes, it.Lk - it.kv0);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(L::kKvFix + kb));
          }
        }
        if (qrow + kBwdTileQ > it.Lq) {
          ok = mbar_wait_warp(bar(L::kQFull + st), ph, abort_flag, kSiteBase + 18);
          ok = ok && mbar_wait_warp(bar(L::kDoFull + st), ph, abort_flag, kSiteBase + 19);
          if (!ok) break;
          zero_rows(smem_gen + L::kQOff + st * kTileBytes, it.Lq - qrow);
          zero_rows(smem_gen + L::kDoOff + st * kTileBytes, it.Lq - qrow);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(L::kQdoFix + st));
        }
      }
      g += it.n_q;
      ++act;
    }
  }
  else if (warp == kBwdIssuerA) {
    // ============================================================ issuer A: S^T = K Q^T, dP^T = V dO^T
    const bool leader = elect_one();
    constexpr uint32_t idesc_st = make_idesc(128, 128, kBF16, false, false);
    constexpr uint32_t kStageStep = kTileBytes >> 4;
    // operands with rows = M / N and the 64 contiguous elements = contraction
    const uint64_t k_km = smem_desc_sw128(smem_base + L::kKOff, 16, 1024);
    const uint64_t v_km = smem_desc_sw128(smem_base + L::kVOff, 16, 1024);
    const uint64_t q_km0 = smem_desc_sw128(smem_base + L::kQOff, 16, 1024);
    const uint64_t do_km0 = smem_desc_sw128(smem_base + L::kDoOff, 16, 1024);
    const uint32_t k_lo = (uint32_t)k_km, v_lo = (uint32_t)v_km, q_lo0 = (uint32_t)q_km0, do_lo0 = (uint32_t)do_km0;
    const uint32_t hi = (uint32_t)(k_km >> 32);  // identical for all four (same layout parameters)
    auto issue = [&](uint32_t dcol, uint32_t a_lo, uint32_t b_lo) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t off = (uint32_t)(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
        mma_ss(leader, tmem + dcol, make_desc(a_lo + off, hi), make_desc(b_lo + off, hi), idesc_st, kk > 0);
      }
    };
    int g = 0;                // query tiles issued so far (all items)
    int act = 0;              // items with work so far
    uint32_t kvfix_par = 0u;  // bit kb: parity of buffer kb's "padded K rows cleared" (one phase per ragged key tile in it)
    uint32_t qfix_par = 0u;   // bit st: parity of stage st's "padded Q / dO rows cleared"
    bool ok = true;
    for (int k = 0; ok; ++k) {
      BwdItem it;
      const int item = read_item(k, it);
      if (item < 0) break;
      if (it.n_q == 0) continue;
      const int kb = act % L::kKvBufs;
      const uint32_t kv_off = (uint32_t)kb * kStageStep;  // this item's K_j / V_j buffer, in descriptor address units
      ok = mbar_wait_warp(bar(L::kKvFull + kb), (uint32_t)(act / L::kKvBufs) & 1u, abort_flag, kSiteBase + 3);
      if (it.ragged_kv) {
        ok = ok && mbar_wait_warp(bar(L::kKvFix + kb), (kvfix_par >> kb) & 1u, abort_flag, kSiteBase + 20);
        kvfix_par ^= 1u << kb;
      }
      for (int t = 0; t < it.n_q && ok; ++t) {
        const int gt = g + t;
        const int st = gt & 1;
        const uint32_t ph = (uint32_t)(gt >> 1) & 1u;  // parity of the stage's "full" barriers
        const uint32_t prev = (uint32_t)(gt - 1) & 1u;
        ok = mbar_wait_warp(bar(L::kQFull + st), ph, abort_flag, kSiteBase + 4);
        if (t == it.n_q - 1 && it.ragged_last_q) {
          ok = ok && mbar_wait_warp(bar(L::kQdoFix + st), (qfix_par >> st) & 1u, abort_flag, kSiteBase + 21);
          qfix_par ^= 1u << st;
        }
        if constexpr (kTwoS) {
          // this S buffer last held tile g-2: its P^T (read by dV) and then its dQ, until that was drained
          if (gt >= 2) ok = ok && mbar_wait_warp(bar(L::kDqEmpty + sbuf(gt)), spar(gt - 2), abort_flag, kSiteBase + 5);
        } else {
          // the S columns still hold P^T of the previous tile until its dV GEMM has read them
          if (gt > 0) ok = ok && mbar_wait_warp(bar(L::kSFree), prev, abort_flag, kSiteBase + 5);
        }
        if (!ok) break;
        tc_fence_after_sync();
        issue(kColS + 128u * (uint32_t)sbuf(gt), k_lo + kv_off, q_lo0 + (uint32_t)st * kStageStep);
        mma_commit(leader, bar(L::kSFull + sbuf(gt)));
        mma_commit(leader, bar(L::kQEmpty + st));
        ok = mbar_wait_warp(bar(L::kDoFull + st), ph, abort_flag, kSiteBase + 6);
        if (gt > 0) {
          // the dP columns hold dS^T of the previous tile (read by dK) and, when dQ shares them,
          // the previous dQ tile until it has been drained
          ok = ok && mbar_wait_warp(bar(kDqT ? L::kDqEmpty : L::kDpFree), prev, abort_flag, kSiteBase + 7);
        }
        if (!ok) break;
        tc_fence_after_sync();
        issue(kColDp, v_lo + kv_off, do_lo0 + (uint32_t)st * kStageStep);
        mma_commit(leader, bar(L::kDpFull));
        mma_commit(leader, bar(L::kDoEmpty + st));
      }
      if (!ok) break;
      mma_commit(leader, bar(L::kKvEmpty + kb));  // this warp's products no longer read K_j, V_j once they complete
      g += it.n_q;
      ++act;
    }
  } else if (warp == kBwdIssuerB) {
    // ============================================================ issuer B: dV, dK, dQ
    const bool leader = elect_one();
    constexpr uint32_t idesc_acc = make_idesc(128, D, kBF16, false, true);  // A in TMEM, B rows = contraction
    // dQ (M = queries, N = D) or dQ^T (M = D, N = queries): both operands rows = contraction
    constexpr uint32_t idesc_dq = kDqT ? make_idesc(D, 128, kBF16, true, true) : make_idesc(128, D, kBF16, true, true);
    constexpr uint32_t kStageStep = kTileBytes >> 4;
    // operands whose rows are the contraction index; the next 64-column block lies 16 KB further
    const uint64_t k_mn = smem_desc_sw128(smem_base + L::kKOff, 16384, 1024);
    const uint64_t ds_mn = smem_desc_sw128(smem_base + L::kDsOff, 16384, 1024);
    const uint64_t q_mn0 = smem_desc_sw128(smem_base + L::kQOff, 16384, 1024);
    const uint64_t do_mn0 = smem_desc_sw128(smem_base + L::kDoOff, 16384, 1024);
    const uint32_t k_lo = (uint32_t)k_mn, ds_lo = (uint32_t)ds_mn, q_lo0 = (uint32_t)q_mn0, do_lo0 = (uint32_t)do_mn0;
    const uint32_t hi = (uint32_t)(k_mn >> 32);
    // acc[key, d] (+)= A^T[key, query] (16-bit, TMEM) . B[query, d]
    auto issue_acc = [&](uint32_t dcol, uint32_t acol, uint32_t b_lo, uint32_t acc0) {
#pragma unroll
      for (int kk = 0; kk < kBwdTileQ / 16; ++kk) {
        // queries 32c .. 32c+31 sit, 16-bit packed, in columns 32c + [0,16) of the source
        mma_ts(leader, tmem + dcol, tmem + acol + 32 * (kk >> 1) + 8 * (kk & 1), make_desc(b_lo + kk * (2048 >> 4), hi),
               idesc_acc, kk > 0 ? 1u : acc0);
      }
    };
    int g = 0;    // query tiles issued so far (all items)
    int act = 0;  // items with work so far
    // who reads the accumulators of an item (0: compute warps, 1: drain warps), for the previous item, and the
    // parity of each of the two hand-back barriers' next phase
    int prev_kind = 0;
    uint32_t empty_par = 0u;  // bit kind
    bool ok = true;
    for (int k = 0; ok; ++k) {
      BwdItem it;
      const int item = read_item(k, it);
      if (item < 0) break;
      if (it.n_q == 0) continue;
      const int kb = act % L::kKvBufs;
      const uint32_t kv_off = (uint32_t)kb * kStageStep;
      ok = mbar_wait_warp(bar(L::kKvFull + kb), (uint32_t)(act / L::kKvBufs) & 1u, abort_flag, kSiteBase + 24);  // K_j for dQ
      // the accumulators still hold the previous item's dK, dV until its epilogue has read them
      if (ok && act > 0) {
        ok = mbar_wait_warp(bar(L::kDkvEmpty + prev_kind), (empty_par >> prev_kind) & 1u, abort_flag, kSiteBase + 33);
        empty_par ^= 1u << prev_kind;
      }
      prev_kind = (kDrainWarps && it.n_q <= kDrainEpilogueMaxTiles) ? 1 : 0;
      for (int t = 0; t < it.n_q && ok; ++t) {
        const int gt = g + t;
        const int st = gt & 1;
        const uint32_t par = (uint32_t)gt & 1u;
        const uint32_t acc0 = t > 0 ? 1u : 0u;
        // dV += P^T dO.  The probabilities only prove that Q_i has landed (they come from S^T = K Q^T): this
        // product is the first of this warp's to read dO_i and waits for that tile itself - without it a row
        // of the stage could still hold the tile of two steps earlier (seen once in some hundred runs on one
        // shape, as dV rows carrying dO of query q - 256 instead of q).
        ok = mbar_wait_warp(bar(L::kDoFull + st), (uint32_t)(gt >> 1) & 1u, abort_flag, kSiteBase + 22);
        ok = ok && mbar_wait_warp(bar(L::kPReady + sbuf(gt)), spar(gt), abort_flag, kSiteBase + 8);
        if (!ok) break;
        tc_fence_after_sync();
        issue_acc(kColDv, kColS + 128u * (uint32_t)sbuf(gt), do_lo0 + (uint32_t)st * kStageStep, acc0);
        if (!kTwoS) mma_commit(leader, bar(L::kSFree));
        mma_commit(leader, bar(L::kDoEmpty + st));
        // dK += dS^T Q  (no wait for Q_i of this warp's own: dS exists only because S^T = K Q^T was computed
        // from the landed tile, so its arrival precedes the barrier below)
        ok = mbar_wait_warp(bar(L::kDsReady), par, abort_flag, kSiteBase + 9);
        if (!ok) break;
        tc_fence_after_sync();
        if constexpr (kTwoS) {
          // dQ first: the compute warps wait for it before they rewrite the shared-memory copy of dS, its
          // drain starts earlier, and at the last tile of an item it is complete before dK is, so that the
          // epilogue may use the dS buffer as scratch as soon as dK_j, dV_j are complete
#pragma unroll
          for (int kk = 0; kk < kBwdTileKV / 16; ++kk) {
            const uint64_t kd = make_desc(k_lo + kv_off + kk * (2048 >> 4), hi), dsd = make_desc(ds_lo + kk * (2048 >> 4), hi);
            mma_ss(leader, tmem + dq_col(gt), dsd, kd, idesc_dq, kk > 0);
          }
          mma_commit(leader, bar(L::kDqFull + sbuf(gt)));
        }
        issue_acc(kColDk, kColDp, q_lo0 + (uint32_t)st * kStageStep, acc0);
        if (!kDqT) mma_commit(leader, bar(L::kDpFree));
        mma_commit(leader, bar(L::kQEmpty + st));
        // dK_j, dV_j are complete with the last tile's dK: the epilogue need not wait for its dQ
        if (t == it.n_q - 1) mma_commit(leader, bar(L::kDkvFull));
        if constexpr (!kTwoS) {
          // the dQ GEMM needs the previous dQ tile read out of its columns
          ok = mbar_wait_warp(bar(L::kDqEmpty), par ^ 1u, abort_flag, kSiteBase + 10);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < kBwdTileKV / 16; ++kk) {
            const uint64_t kd = make_desc(k_lo + kv_off + kk * (2048 >> 4), hi), dsd = make_desc(ds_lo + kk * (2048 >> 4), hi);
            mma_ss(leader, tmem + dq_col(gt), kDqT ? kd : dsd, kDqT ? dsd : kd, idesc_dq, kk > 0);
          }
          mma_commit(leader, bar(L::kDqFull + sbuf(gt)));
        }
      }
      if (!ok) break;
      mma_commit(leader, bar(L::kKvEmpty + kb));  // the dQ products were this warp's readers of K_j
      g += it.n_q;
      ++act;
    }
  }
  else if (warp < kBwdComputeWarps) {
    // ============================================================ compute warps
    const int quarter = warp & 3;                         // TMEM lane quarter this warp may access
    const int cg = warp >> 2;                             // query-column group: columns 32 cg .. 32 cg + 31
    const int lane_row = quarter * 32 + lane;             // key row within the tile == TMEM lane
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_addr0 = tmem + lane_addr + kColS + 32 * cg;  // + 128 for the second S buffer
    const uint32_t dp_addr = tmem + lane_addr + kColDp + 32 * cg;
    const float c1 = p.scale * kLog2e;
    // shared-memory copy of dS^T: [2 blocks of 64 queries][128 key rows][128 bytes], 128-byte swizzle
    const uint32_t ds_line = smem_base + L::kDsOff + (cg >> 1) * 16384 + lane_row * 128;
    const uint32_t chunk0 = (uint32_t)(cg & 1) * 4;
    const uint32_t sw = (uint32_t)(lane_row & 7);
    // D = 128: lane l of quarter k holds d = 32 k + l of dQ^T; this warp takes query columns 32 cg ..
    // D = 64:  this thread holds query row `lane_row`, head columns 16 cg .. 16 cg + 15 of dQ
    const uint32_t dq_off = tmem + lane_addr + (kDqT ? 32 : 16) * cg;
    int g = 0;    // query tiles processed so far (all items)
    int act = 0;  // items with work so far
    bool ok = true;

    for (int k = 0; ok; ++k) {
      BwdItem it;
      const int item = read_item(k, it);
      if (item < 0) break;
      const int b = it.b, h = it.h, kv0 = it.kv0, Lq = it.Lq, Lk = it.Lk, i_begin = it.i_begin, n_q = it.n_q;
      const int kv = kv0 + lane_row;
      if (n_q == 0) {
        // no query sees this key tile: its gradients are zero
        uint8_t* dk_base = reinterpret_cast<uint8_t*>(p.dk) +
                           2 * ((int64_t)it.bc * p.dk_sb + (int64_t)h * p.dk_sh + (int64_t)it.tk0 * p.dk_st);
        uint8_t* dv_base = reinterpret_cast<uint8_t*>(p.dv) +
                           2 * ((int64_t)it.bc * p.dv_sb + (int64_t)h * p.dv_sh + (int64_t)it.tk0 * p.dv_st);
        constexpr int kChunksPerRow = D * 2 / 16;
        for (int i = threadIdx.x; i < kBwdTileKV * kChunksPerRow; i += kBwdComputeWarps * 32) {
          const int row = kv0 + i / kChunksPerRow;
          if (row < it.key_lim) {
            *reinterpret_cast<uint4*>(dk_base + 2 * (int64_t)row * p.dk_st + 16 * (i % kChunksPerRow)) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(dv_base + 2 * (int64_t)row * p.dv_st + 16 * (i % kChunksPerRow)) = make_uint4(0, 0, 0, 0);
          }
        }
        continue;
      }
      float c0 = it.bias;
      if (p.score_mod && kv < it.key_lim) c0 += p.score_mod[(p.cu_k ? (int64_t)it.tk0 : (int64_t)b * p.Tk) + kv];
      c0 *= kLog2e;
      const bool row_ok = kv < Lk;

      // ---- dQ drain (see the file header); t = index within the item of the query tile whose dQ is complete
      // ---- dQ^T drain by the compute warps themselves (D = 128; at D = 64 the drain warps do it): lane l of
      // quarter k holds d = 32 k + l, this warp takes query columns 32 cg ..; one red.global.add.f32 per
      // query covers a full 128-byte line.  t = index within the item of the query tile whose dQ is complete
      auto drain_dq = [&](int t) {
        const int gt = g + t;
        ok = mbar_wait_warp(bar(L::kDqFull + sbuf(gt)), spar(gt), abort_flag, kSiteBase + 14);
        const uint32_t dq_addr = dq_off + dq_col(gt);
        if (!ok) return;
        tc_fence_after_sync();
        const int q_tile = (i_begin + t) * kBwdTileQ;
        uint32_t r[32];
        tmem_ld32_sync(dq_addr, r);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(L::kDqEmpty + sbuf(gt)));  // the TMEM columns are free again
        const int q_first = q_tile + 32 * cg;
        float* dst = p.dq_acc + ((it.acc_row0 + q_first) * p.H + h) * D + lane_row;
        const int64_t row_stride = (int64_t)p.H * D;
        const int n_live = min(32, Lq - q_first);  // queries at or beyond Lq get no gradient
#pragma unroll
        for (int v = 0; v < 32; ++v) {
          if (v < n_live)
            asm volatile("red.global.add.f32 [%0], %1;" ::"l"(dst + v * row_stride), "f"(__uint_as_float(r[v])) : "memory");
        }
      };

      for (int t = 0; t < n_q; ++t) {
        const int gt = g + t;
        const int q0 = (i_begin + t) * kBwdTileQ + 32 * cg;  // first query index of my columns
        // valid queries for this key row: q_lo <= q < q_hi (empty when the key row is padding)
        const int q_lo = p.causal ? kv : 0;
        const int q_hi = row_ok ? Lq : 0;
        // warp-uniform on purpose: the two instantiations contain warp-collective TMEM accesses
        const bool need_mask = it.ragged_kv || (q0 + 32 > Lq) || (p.causal && q0 < kv0 + kBwdTileKV - 1);
        float pv[32];
        ok = mbar_wait_warp(bar(L::kSFull + sbuf(gt)), spar(gt), abort_flag, kSiteBase + 12);
        const uint32_t s_addr = s_addr0 + 128u * (uint32_t)sbuf(gt);
        if (!ok) break;
        tc_fence_after_sync();
        if constexpr (kDrainWarps) {
          if (need_mask) bwd_phase_a16<kBF16, true, kAccurate>(s_addr, c1, c0, q0, q_lo, q_hi);
          else           bwd_phase_a16<kBF16, false, kAccurate>(s_addr, c1, c0, q0, q_lo, q_hi);
        } else {
          if (need_mask) bwd_phase_a<kBF16, true, kAccurate>(s_addr, c1, c0, q0, q_lo, q_hi, pv);
          else           bwd_phase_a<kBF16, false, kAccurate>(s_addr, c1, c0, q0, q_lo, q_hi, pv);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(L::kPReady + sbuf(gt)));

        if constexpr (kDrainWarps) {
          // the dQ product of the previous tile (of this or the previous item) reads the shared-memory copy
          // of dS until it is complete; phase B below rewrites that copy
          if (gt > 0) ok = mbar_wait_warp(bar(L::kDqFull + sbuf(gt - 1)), spar(gt - 1), abort_flag, kSiteBase + 16);
          if (!ok) break;
        } else if (t > 0) {
          // dQ of the previous tile is complete by now (or soon): drain it while dP^T is computed.
          // Its completion also means the dQ GEMM no longer reads the shared-memory copy of dS.
          drain_dq(t - 1);
          if (!ok) break;
        }

        ok = mbar_wait_warp(bar(L::kDpFull), (uint32_t)gt & 1u, abort_flag, kSiteBase + 13);
        if (!ok) break;
        tc_fence_after_sync();
        if constexpr (kDrainWarps) {
          if (need_mask) bwd_phase_b16<kBF16, true>(s_addr, dp_addr, ds_line, chunk0, sw);
          else           bwd_phase_b16<kBF16, false>(s_addr, dp_addr, ds_line, chunk0, sw);
        } else {
          if (need_mask) bwd_phase_b<kBF16, true>(dp_addr, ds_line, chunk0, sw, pv);
          else           bwd_phase_b<kBF16, false>(dp_addr, ds_line, chunk0, sw, pv);
        }
        fence_proxy_async_smem();
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(L::kDsReady));
      }
      if (!ok) break;

      // ------------------------------------------------------------ epilogue of the item
      // (before the drain of the last dQ tile, whose product is still running); short items' at D = 64 is the
      // drain warps' (kDrainEpilogueMaxTiles): nothing of the accumulators is needed here then
      // column groups 0,1 store dV, groups 2,3 store dK (each half of the head dimension)
      if (kDrainWarps && n_q <= kDrainEpilogueMaxTiles) {
        // (no arrival either: each of the two hand-back barriers is arrived on only by the warps that read the
        // accumulators of that item - a group that runs ahead must not add arrivals to a phase that still
        // waits for the other group's)
      } else {
      ok = mbar_wait_warp(bar(L::kDkvFull), (uint32_t)act & 1u, abort_flag, kSiteBase + 15);
      if (!ok) break;
      {
        tc_fence_after_sync();
        const bool is_dk = cg >= 2;
        const int col0 = (cg & 1) * (D / 2);
        const uint32_t acc_addr = tmem + lane_addr + (is_dk ? kColDk : kColDv) + col0;
        const float mul = is_dk ? p.scale : 1.0f;
        // out of TMEM already rounded to 16 bits, so that few registers are live across the hand-over
        uint4 w[D / 64][4];
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          uint32_t r[32];
          tmem_ld32_sync(acc_addr + c * 32, r);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            w[c][q4].x = pack2<kBF16>(mul * __uint_as_float(r[8 * q4 + 0]), mul * __uint_as_float(r[8 * q4 + 1]));
            w[c][q4].y = pack2<kBF16>(mul * __uint_as_float(r[8 * q4 + 2]), mul * __uint_as_float(r[8 * q4 + 3]));
            w[c][q4].z = pack2<kBF16>(mul * __uint_as_float(r[8 * q4 + 4]), mul * __uint_as_float(r[8 * q4 + 5]));
            w[c][q4].w = pack2<kBF16>(mul * __uint_as_float(r[8 * q4 + 6]), mul * __uint_as_float(r[8 * q4 + 7]));
            if (!row_ok) w[c][q4] = make_uint4(0, 0, 0, 0);
          }
        }
        // the accumulators are in registers: the next item's first dV / dK products may overwrite them
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(L::kDkvEmpty + 0));
        // row 0 of this sequence's dK or dV, at this warp's columns
        const int64_t out_st = is_dk ? p.dk_st : p.dv_st;
        uint8_t* out_base = is_dk ? reinterpret_cast<uint8_t*>(p.dk) + 2 * ((int64_t)it.bc * p.dk_sb + (int64_t)h * p.dk_sh + (int64_t)it.tk0 * p.dk_st)
                                  : reinterpret_cast<uint8_t*>(p.dv) + 2 * ((int64_t)it.bc * p.dv_sb + (int64_t)h * p.dv_sh + (int64_t)it.tk0 * p.dv_st);
        out_base += 2 * col0;
        if constexpr (D == 64) {
          // A lane holds 64 bytes of its key row; written as they are, one store instruction would touch 32
          // lines (the load/store unit takes them one at a time: about 2000 clocks per item for the CTA).
          // Each warp therefore turns its 32 x 64-byte block through its own part of the shared-memory copy
          // of dS - the rows and 16-byte slots it writes in phase B, which no product reads any more once
          // the item's last dK is complete - so that four lanes cover a row and an instruction 8 rows.
          uint8_t* ds_gen = smem_gen + L::kDsOff + (cg >> 1) * 16384 + quarter * 32 * 128;  // row 0 of this warp's quarter
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4)
            *reinterpret_cast<uint4*>(ds_gen + lane * 128 + (((chunk0 + q4) ^ sw) << 4)) = w[0][q4];
          __syncwarp();
          const int c = lane & 3;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r = 8 * i + (lane >> 2);  // row within the quarter (quarter * 32 is a multiple of 8: same swizzle phase)
            const uint4 x = *reinterpret_cast<const uint4*>(ds_gen + r * 128 + (((chunk0 + c) ^ (uint32_t)(r & 7)) << 4));
            const int krow = kv0 + quarter * 32 + r;
            if (krow < it.key_lim) *reinterpret_cast<uint4*>(out_base + 2 * (int64_t)krow * out_st + 16 * c) = x;
          }
          __syncwarp();  // phase B of the next item rewrites these slots
        } else {
          if (kv < it.key_lim) {
            uint8_t* out_row = out_base + 2 * (int64_t)kv * out_st;
#pragma unroll
            for (int c = 0; c < D / 64; ++c) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) *reinterpret_cast<uint4*>(out_row + 64 * c + 16 * q4) = w[c][q4];
            }
          }
        }
      }
      }
      if constexpr (!kDrainWarps) {
        drain_dq(n_q - 1);
        if (!ok) break;
      }
      g += n_q;
      ++act;
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kBwdIssuerA) {
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

// dQ = scale * accumulator, cast to the 16-bit type.  acc is [B, T, H, D] contiguous fp32.
struct DqConvertParams {
  const float* acc;
  void* dq;
  int64_t sb, st, sh;
  int B, T, H;
  float scale;
};

template <int D, bool kBF16>
__global__ void __launch_bounds__(256) sigattn_dq_convert_kernel(const DqConvertParams p) {
  constexpr int kChunks = D / 8;  // 8 elements (16 bytes out, 32 bytes in) per chunk
  const long long total = (long long)p.B * p.T * p.H * kChunks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % kChunks);
    long long r = i / kChunks;
    const int h = (int)(r % p.H);
    r /= p.H;
    const int t = (int)(r % p.T);
    const int b = (int)(r / p.T);
    const float4 a0 = __ldg(reinterpret_cast<const float4*>(p.acc) + 2 * i);
    const float4 a1 = __ldg(reinterpret_cast<const float4*>(p.acc) + 2 * i + 1);
    uint4 w;
    w.x = pack2<kBF16>(a0.x * p.scale, a0.y * p.scale);
    w.y = pack2<kBF16>(a0.z * p.scale, a0.w * p.scale);
    w.z = pack2<kBF16>(a1.x * p.scale, a1.y * p.scale);
    w.w = pack2<kBF16>(a1.z * p.scale, a1.w * p.scale);
    uint8_t* dst = reinterpret_cast<uint8_t*>(p.dq) + 2 * ((int64_t)b * p.sb + (int64_t)t * p.st + (int64_t)h * p.sh) + 16 * c;
    *reinterpret_cast<uint4*>(dst) = w;
  }
}

}  // namespace sigattn
