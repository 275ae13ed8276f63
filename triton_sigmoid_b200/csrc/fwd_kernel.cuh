// Forward kernel: O = sigmoid(scale * Q K^T + bias) V.  A work item is one (batch, head,
// 256-query block); the kernel is persistent: one CTA per SM takes items from a ticket counter
// until none are left, so that loads and scores of the next item overlap the epilogue of the
// current one and uneven items (causal, ragged lengths) balance themselves.
//
// Takes over the work of the reference's _fwd_dense_kernel
// (src/triton_sigmoid/sigmoid_triton_dense.py:23-154) and _fwd_padded_kernel
// (src/triton_sigmoid/sigmoid_triton_padded.py:24-171).
//
// Structure (sm_100a, 24 warps):
//   warps 0-15   sigmoid warps.  A JOB is one query tile (128 rows) times one key tile (128 columns);
//                one thread per row, 32-column chunks, P written over the start of the chunk's columns.
//                D = 128: all sixteen warps work on the same job (warp w: TMEM lanes 32 (w & 3) ..,
//                key columns 32 (w >> 2) ..).  With eight warps per job and two jobs in the sigmoid
//                stage at a time, a score buffer stays occupied for about three job times, and the two
//                buffers TMEM has room for at D = 128 starve the sigmoid warps (measured: 44 % of their
//                time waiting for scores); with sixteen warps per job it is occupied for about two.
//                D = 64: warps 0-7 take the jobs of query tile 0, warps 8-15 those of tile 1 (warp w:
//                lanes 32 (w & 3) .., columns 64 ((w >> 2) & 1) .., two chunks per job, the second
//                loaded while the first is computed); three buffers are enough for that, and the
//                per-job costs (barrier round trip, exposed TMEM load) are paid once per 64 columns
//                (measured faster at D = 64 than sixteen warps per job: 728 against 647 TFLOP/s).
//   warp  16     item scheduler + TMA producer: Q tiles per item, K_j / V_j through a ring of smem stages
//   warp  17     tcgen05 issuer 1: S = Q_s K_j^T (smem x smem -> TMEM fp32); owns the TMEM allocation
//   warp  18     tcgen05 issuer 2: O_s += P V_j (TMEM x smem -> TMEM fp32)
//   warps 20-23  output warps (one per TMEM lane quarter): wait for an item's last P V product, read O out of
//                TMEM, round it and write it to global memory, while the sigmoid warps are already at work
//                on the next item's scores (measured against the sigmoid warps writing O themselves:
//                +8 % at N = 512, +3 % at N = 1024-2048, +1 % at N = 4096); O goes through shared memory
//                so that whole rows leave per instruction (D = 64: the item's two tiles at once, D = 128:
//                one tile at a time)
// There is no row normaliser in sigmoid attention, so O simply accumulates in TMEM over the
// whole key loop of an item.  The (query tile, key tile) jobs are processed in a fixed order through a
// small ring of S buffers in TMEM (3 when D = 64, 2 when D = 128): the issuer computes the
// scores of a later job while the sigmoid warps turn an earlier one into 16-bit P in place
// (each warp writes P over the start of the columns it has just read) and signal the issuer.
//
// Masking: key tiles beyond the causal diagonal or the valid key length are skipped
// entirely; tiles that straddle either boundary apply an element predicate.
#pragma once

#include "ptx.cuh"
#include "sigmoid_math.cuh"

namespace sigattn {

struct FwdParams {
  void* o;
  int64_t o_sb, o_st, o_sh;  // element strides of O: batch, token, head
  const int* lens_q;
  const int* lens_k;
  // Packed (variable-length) layout: sequence b occupies rows cu_q[b] .. cu_q[b+1]-1 of a (total, H, D)
  // tensor (likewise cu_k for keys / values); Tq, Tk are then upper bounds of the lengths.  nullptr = (B, T, H, D).
  const int* cu_q;
  const int* cu_k;
  const float* bias;       // [B] or nullptr
  const float* score_mod;  // [B, Tk] (packed: [total keys]) or nullptr
  float scale;
  float bias_scalar;
  int B, H, Tq, Tk;
  int causal;
  int n_qblk;   // ceil(Tq / 256)
  int n_items;  // B * H * n_qblk
  int group;    // (batch, head) pairs per scheduling group, >= 1 (see fwd_decode_item)
  // two counters, zero between launches: [0] items handed out beyond the first per CTA,
  // [1] CTAs that have finished (the last one clears both)
  unsigned int* ticket;
};

constexpr int kFwdSigmoidWarps = 16;
constexpr int kFwdProducerWarp = kFwdSigmoidWarps;
constexpr int kFwdIssuerWarp = kFwdSigmoidWarps + 1;   // S = Q K^T, owns the TMEM allocation
constexpr int kFwdIssuerWarp2 = kFwdSigmoidWarps + 2;  // O += P V
constexpr int kFwdOutputWarp0 = kFwdSigmoidWarps + 4;  // four output warps, one per TMEM lane quarter
constexpr int kFwdThreads = (kFwdSigmoidWarps + 8) * 32;  // role warps and output warps: two register-allocation groups of four
constexpr int kFwdLaunchRegs = 80;  // what 768 threads per CTA get each: 65536 / 768, rounded down to a multiple of 8
// Registers per thread after the re-allocation: the role warps, the output warps (a group of four each)
// and the sigmoid warps.
template <int D> struct FwdRegs {
  static constexpr int kRole = 48;
  static constexpr int kOutput = 48;
  static constexpr int kSigmoid = 96;
  static_assert(kFwdSigmoidWarps * 32 * kSigmoid + 128 * kRole + 128 * kOutput <= kFwdThreads * kFwdLaunchRegs,
                "the re-allocation may not ask for more registers than the CTA holds");
};
constexpr int kFwdBlockM = 256;  // query rows per CTA (two 128-row tiles)
constexpr int kTileN = 128;      // key rows per step

template <int D>
struct FwdSmem {
  static constexpr int kStages = (D == 64) ? 4 : 2;
  static constexpr int kSBufs = (D == 64) ? 3 : 2;  // S buffers in TMEM
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + 2 * kTileBytes;
  static constexpr int kVOff = kKOff + kStages * kTileBytes;
  // staging for the output warps, 8 KB each: D = 64 a whole item's O (2 query tiles x 32 rows x 128 bytes),
  // D = 128 one query tile at a time (32 rows x 256 bytes)
  static constexpr int kOutOff = kVOff + kStages * kTileBytes;
  static constexpr int kOutBytes = 4 * 8192;
  static constexpr int kBarOff = kOutOff + kOutBytes;
  // barrier slots (8 bytes each)
  static constexpr int kQFull = 0;                    // [2]
  static constexpr int kKFull = kQFull + 2;           // [kStages]
  static constexpr int kKEmpty = kKFull + kStages;    // [kStages]
  static constexpr int kVFull = kKEmpty + kStages;    // [kStages]
  static constexpr int kVEmpty = kVFull + kStages;    // [kStages]
  static constexpr int kSFull = kVEmpty + kStages;    // [kSBufs]
  static constexpr int kPFull = kSFull + kSBufs;      // [kSBufs]
  static constexpr int kOFull = kPFull + kSBufs;      // [1]
  static constexpr int kVFix = kOFull + 1;            // [kStages] padded rows of the stage's V tile zeroed
  static constexpr int kPvDone = kVFix + kStages;     // [kSBufs] P V product of the buffer's job complete
  static constexpr int kQEmpty = kPvDone + kSBufs;    // [1] all score products of the item issued and complete
  static constexpr int kOEmpty = kQEmpty + 1;         // [1] O of the item read out of TMEM
  static constexpr int kItemFull = kOEmpty + 1;       // [2] item index published
  static constexpr int kItemEmpty = kItemFull + 2;    // [2] item index read by every consumer warp
  static constexpr int kNumBars = kItemEmpty + 2;
  static constexpr int kMiscOff = kBarOff + 8 * kNumBars;  // tmem base (u32), abort flag (int), 2 x item record (16 int each)
  static constexpr int kTotal = kMiscOff + 16 + 2 * 64;
  static constexpr int kDynBytes = kTotal + 1024;  // slack to align the base to 1024 bytes
};

// Cursor over the job order (0,0) (1,0) (0,1) (1,1) ... restricted to j < n_kv[s], with
// everything an issuing warp needs about the job carried along incrementally.
struct FwdCursor {
  int s, j;     // query tile, key tile
  int st;       // smem stage of key tile j
  uint32_t ph;  // parity of that stage's "full" barrier
  int buf;      // S buffer of the job
  uint32_t bph; // parity of that buffer's barriers
  bool fresh;   // first job that touches key tile j
  // start of a new item: stage and buffer positions carry over from the previous item
  __device__ __forceinline__ void begin_item(int n0) {
    s = (n0 > 0) ? 0 : 1;
    j = 0;
    fresh = true;
  }
  __device__ __forceinline__ void advance(int n0, int n1, int n_stages, int n_bufs) {
    if (s == 0 && j < n1) {
      s = 1;
      fresh = false;
    } else {
      ++j;
      s = (j < n0) ? 0 : 1;
      if (++st == n_stages) { st = 0; ph ^= 1u; }
      fresh = true;
    }
    if (++buf == n_bufs) { buf = 0; bph ^= 1u; }
  }
};

// 32 score columns of one TMEM lane (this thread's query row), already in registers -> logits in the
// base-2 domain, t = (scale * s + bias (+ score_mod[key])) * log2(e).  Chunks that need no element
// predicate work on logits shifted up by kDeepShift (see sigmoid2_from_shifted_log2_deep).
// col0 = key index of the first column.
template <bool kScoreMod, bool kMask, bool kAccurate>
__device__ __forceinline__ void fwd_chunk_logits(const uint32_t (&r)[32], float2 (&t)[16], float c1, float c0, int col0,
                                                 const float* sm_row, int Tk) {
  constexpr int kCh = 32;
  constexpr bool kShift = !kMask && !kAccurate;
  const float c0s = kShift ? c0 + kDeepShift : c0;
#pragma unroll
  for (int i = 0; i < kCh / 2; ++i) {
    t[i] = __ffma2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), make_float2(c1, c1),
                      make_float2(c0s, c0s));
  }
  if constexpr (kScoreMod) {
    // per-key additive bias: the same value for every lane (row), read through the read-only path
    if (col0 + kCh <= Tk && (reinterpret_cast<uintptr_t>(sm_row + col0) & 15u) == 0) {
#pragma unroll
      for (int i = 0; i < kCh / 4; ++i) {
        const float4 m = __ldg(reinterpret_cast<const float4*>(sm_row + col0) + i);
        t[2 * i] = __ffma2_rn(make_float2(m.x, m.y), make_float2(kLog2e, kLog2e), t[2 * i]);
        t[2 * i + 1] = __ffma2_rn(make_float2(m.z, m.w), make_float2(kLog2e, kLog2e), t[2 * i + 1]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < kCh / 2; ++i) {
        const int col = col0 + 2 * i;
        t[i].x = fmaf(col < Tk ? __ldg(sm_row + col) : 0.0f, kLog2e, t[i].x);
        t[i].y = fmaf(col + 1 < Tk ? __ldg(sm_row + col + 1) : 0.0f, kLog2e, t[i].y);
      }
    }
  }
}

// Logits of fwd_chunk_logits -> 16-bit probabilities, written over the first 16 of the chunk's 32 TMEM
// columns at s_addr.  lim = largest visible key index of this row (used only when kMask).
template <bool kBF16, bool kMask, bool kAccurate>
__device__ __forceinline__ void fwd_chunk_probs(uint32_t s_addr, float2 (&t)[16], int col0, int lim) {
  constexpr int kCh = 32;
  uint32_t pk[kCh / 2];
  if constexpr (kAccurate) {
#pragma unroll
    for (int i = 0; i < kCh / 2; ++i) {
      float2 pr = sigmoid2_accurate_from_log2(t[i]);
      if constexpr (kMask) {
        const int col = col0 + 2 * i;
        pr.x = (col <= lim) ? pr.x : 0.0f;
        pr.y = (col + 1 <= lim) ? pr.y : 0.0f;
      }
      pk[i] = pack2<kBF16>(pr.x, pr.y);
    }
  } else {
    // Under the default bias every logit of a chunk is far below zero: the short series applies
    // and the sign handling (one compare and one select per element) is skipped for the whole warp.
    if (!kMask && warp_all_negative(t)) {
#pragma unroll
      for (int i = 0; i < kCh / 2; ++i) pk[i] = sigmoid2_deep_packed<kBF16>(t[i], (i & 7) == 7);
    } else {
      bool all_neg = false;
      if constexpr (!kMask) {
#pragma unroll
        for (int i = 0; i < kCh / 2; ++i) t[i] = __fadd2_rn(t[i], make_float2(-kDeepShift, -kDeepShift));
        all_neg = warp_all_negative(t);  // negative but not far below zero: full polynomial, still no select
      }
      if (all_neg) {
#pragma unroll
        for (int i = 0; i < kCh / 2; ++i) {
          const float2 pr = sigmoid2_from_log2_neg<kBF16>(t[i]);
          pk[i] = pack2<kBF16>(pr.x, pr.y);
        }
      } else {
#pragma unroll
        for (int i = 0; i < kCh / 2; ++i) {
          float2 pr = sigmoid2_from_log2<kBF16>(t[i]);
          if constexpr (kMask) {
            const int col = col0 + 2 * i;
            pr.x = (col <= lim) ? pr.x : 0.0f;
            pr.y = (col + 1 <= lim) ? pr.y : 0.0f;
          }
          pk[i] = pack2<kBF16>(pr.x, pr.y);
        }
      }
    }
  }
  tmem_st(s_addr, pk);
}

// Both steps for a chunk whose scores are in registers.
template <bool kBF16, bool kScoreMod, bool kMask, bool kAccurate>
__device__ __forceinline__ void fwd_sigmoid_chunk(uint32_t s_addr, const uint32_t (&r)[32], float c1, float c0, int col0,
                                                  int lim, const float* sm_row, int Tk) {
  float2 t[16];
  fwd_chunk_logits<kScoreMod, kMask, kAccurate>(r, t, c1, c0, col0, sm_row, Tk);
  fwd_chunk_probs<kBF16, kMask, kAccurate>(s_addr, t, col0, lim);
}

// One work item.  The producer warp decodes it once (integer divisions, length and bias loads from global
// memory) and publishes the record through shared memory; every other role reads it from there - decoding
// in each of the eighteen consumer warps cost the sigmoid warps about two thousand clocks per item.
struct FwdItem {
  int b, h, q0;
  int bc;             // batch coordinate of the tensor maps and strides (0 when packed)
  int tq0, tk0;       // first row of the sequence in the token dimension (0 unless packed)
  int row_lim;        // query rows below this are written (Tq; packed: Lq, the next rows belong to another sequence)
  int key_lim;        // keys below this have a score_mod entry (Tk; packed: Lk)
  int Lq, Lk;
  int n0, n1, n_max;  // key tiles of query tile 0 / 1, and the larger of the two
  float bias;         // additive bias of the item's batch element
};
// record layout in shared memory: 16 ints, [0] = item index (-1: no more work)
__device__ __forceinline__ void fwd_publish_item(volatile int* rec, int item, const FwdItem& it) {
  rec[1] = it.b; rec[2] = it.h; rec[3] = it.q0; rec[4] = it.bc; rec[5] = it.tq0; rec[6] = it.tk0;
  rec[7] = it.row_lim; rec[8] = it.key_lim; rec[9] = it.Lq; rec[10] = it.Lk; rec[11] = it.n0; rec[12] = it.n1;
  rec[13] = it.n_max; rec[14] = __float_as_int(it.bias);
  rec[0] = item;
}
__device__ __forceinline__ FwdItem fwd_load_item(const volatile int* rec) {
  FwdItem it;
  it.b = rec[1]; it.h = rec[2]; it.q0 = rec[3]; it.bc = rec[4]; it.tq0 = rec[5]; it.tk0 = rec[6];
  it.row_lim = rec[7]; it.key_lim = rec[8]; it.Lq = rec[9]; it.Lk = rec[10]; it.n0 = rec[11]; it.n1 = rec[12];
  it.n_max = rec[13]; it.bias = __int_as_float(rec[14]);
  return it;
}
__device__ __forceinline__ FwdItem fwd_decode_item(const FwdParams& p, int item) {
  FwdItem it;
  // Items are ordered in groups of `group` (batch, head) pairs: within a group all pairs' heaviest
  // query blocks come first, then their second heaviest, ... (a longest-first order under a causal
  // mask, which the ticket counter turns into a balanced schedule), while the K / V of one group
  // still fit the L2.  group = 1 is plain (batch, head)-major order.
  const int per_group = p.group * p.n_qblk;
  const int grp = item / per_group;
  const int r = item - grp * per_group;
  const int g_eff = min(p.group, p.B * p.H - grp * p.group);
  const int qi = r / g_eff;
  const int bh = grp * p.group + (r - qi * g_eff);
  it.b = bh / p.H;
  it.h = bh - it.b * p.H;
  const int qblk = p.causal ? (p.n_qblk - 1 - qi) : qi;  // heavy blocks of a head first
  it.q0 = qblk * kFwdBlockM;
  it.Lq = p.Tq;
  it.Lk = p.Tk;
  if (p.lens_q) it.Lq = min(max(p.lens_q[it.b], 0), p.Tq);
  if (p.lens_k) it.Lk = min(max(p.lens_k[it.b], 0), p.Tk);
  it.bc = it.b;
  it.tq0 = it.tk0 = 0;
  it.row_lim = p.Tq;
  it.key_lim = p.Tk;
  if (p.cu_q) {
    it.tq0 = p.cu_q[it.b];
    it.tk0 = p.cu_k[it.b];
    it.Lq = min(max(p.cu_q[it.b + 1] - it.tq0, 0), p.Tq);
    it.Lk = min(max(p.cu_k[it.b + 1] - it.tk0, 0), p.Tk);
    it.bc = 0;
    it.row_lim = it.Lq;
    it.key_lim = it.Lk;
  }
  int n_kv[2];
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const int r0 = it.q0 + 128 * s;
    int kv_end = it.Lk;
    if (p.causal) kv_end = min(kv_end, r0 + 128);
    n_kv[s] = (r0 < it.Lq) ? (kv_end + kTileN - 1) / kTileN : 0;
  }
  it.n0 = n_kv[0];
  it.n1 = n_kv[1];
  it.n_max = max(it.n0, it.n1);
  it.bias = item_bias(p.bias, p.bias_scalar, it.b, it.Lk);
  return it;
}

template <int D, bool kBF16, bool kScoreMod, bool kAccurate>
__global__ void __launch_bounds__(kFwdThreads, 1)
sigattn_fwd_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                   const __grid_constant__ CUtensorMap v_map, const FwdParams p) {
  using L = FwdSmem<D>;
  constexpr int kStages = L::kStages;
  constexpr int kSBufs = L::kSBufs;
  constexpr int kTileBytes = L::kTileBytes;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0;              // S buffer i at kColS + 128 i
  constexpr uint32_t kColO = 128 * kSBufs;   // O_s at kColO + D s
  constexpr int kSiteBase = 0x10000;
  constexpr int kJobWarps = (D == 64) ? 8 : 16;  // sigmoid warps per job (see the file header)
  // warps that read the published item record: the sigmoid warps, the two issuing warps, the output warps
  constexpr int kItemReaders = kFwdSigmoidWarps + 2 + 4;
  static_assert(kColO + 2 * D <= kTmemCols, "TMEM budget");

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
    mbar_init(bar(L::kQFull + 0), 1);
    mbar_init(bar(L::kQFull + 1), 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar(L::kKFull + i), 1);
      mbar_init(bar(L::kKEmpty + i), 1);
      mbar_init(bar(L::kVFull + i), 1);
      mbar_init(bar(L::kVEmpty + i), 1);
    }
    for (int i = 0; i < kSBufs; ++i) {
      mbar_init(bar(L::kSFull + i), 1);
      mbar_init(bar(L::kPFull + i), kJobWarps);  // one arrival per sigmoid warp of the job
      mbar_init(bar(L::kPvDone + i), 1);
    }
    mbar_init(bar(L::kOFull), 1);
    for (int i = 0; i < kStages; ++i) mbar_init(bar(L::kVFix + i), 1);
    mbar_init(bar(L::kQEmpty), 1);
    mbar_init(bar(L::kOEmpty), 4);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(L::kItemFull + i), 1);
      mbar_init(bar(L::kItemEmpty + i), kItemReaders);
    }
    fence_mbar_init();
  }
  if (warp == kFwdProducerWarp && lane == 0) {
    tma_prefetch_desc(&q_map);
    tma_prefetch_desc(&k_map);
    tma_prefetch_desc(&v_map);
  }
  if (warp == kFwdIssuerWarp) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  // The sigmoid warps hold 64 scores each in flight and want more registers than an even split
  // gives; the role warps and the output warps need few.  Registers only move within what the CTA was
  // given at launch, so the counts must add up to no more than that (else the increase never returns).

  // Consumer side of the item ring: returns the k-th item of this CTA, or -1 when there is none
  // (also on a failed wait).  Called by all 32 lanes of a reader warp.
  auto read_item = [&](int k, FwdItem& it) -> int {
    const int slot = k & 1;
    if (!mbar_wait_warp(bar(L::kItemFull + slot), (uint32_t)(k >> 1) & 1u, abort_flag, kSiteBase + 30)) return -1;
    const int item = item_ring[16 * slot];
    if (item >= 0) it = fwd_load_item(item_ring + 16 * slot);
    __syncwarp();
    if (lane == 0) mbar_arrive(bar(L::kItemEmpty + slot));
    return item;
  };

  if (warp >= kFwdOutputWarp0) {
    // ============================================================ output warps: O from TMEM to global memory
    // Four warps, one per TMEM lane quarter (a warp can only read the lanes 32 (warp % 4) ..), one thread
    // per query row.  They take the finished accumulators of an item off the sigmoid warps' hands: those go
    // straight on to the next item's scores while the last P V products complete and O is written out.
    setmaxnreg_dec<FwdRegs<D>::kOutput>();
    const int lane_row = (warp & 3) * 32 + lane;
    const uint32_t tmem_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    int act = 0;  // items with work so far
    bool ok = true;
    for (int k = 0; ok; ++k) {
      const int islot = k & 1;
      ok = mbar_wait_warp(bar(L::kItemFull + islot), (uint32_t)(k >> 1) & 1u, abort_flag, kSiteBase + 30);
      if (!ok) break;
      const volatile int* rec = item_ring + 16 * islot;
      if (rec[0] < 0) break;
      const FwdItem it = fwd_load_item(rec);
      if (it.n_max > 0) {
        ok = mbar_wait_warp(bar(L::kOFull), (uint32_t)act & 1u, abort_flag, kSiteBase + 12);
        if (!ok) break;
        ++act;
        tc_fence_after_sync();
      }
      if constexpr (D == 64) {
        // The whole item's O goes through shared memory: out of TMEM one row per lane (two 16-column loads in
        // flight at a time), rounded to 16 bits, into this warp's patches (16-byte chunks swizzled by row, so
        // neither side has bank conflicts).  The accumulators are handed back as soon as the last load has
        // landed - the next item's first P V product waits for that - and only then the rows go out to global
        // memory, eight lanes per 128-byte row, four rows per instruction.
        uint8_t* stage = smem_gen + L::kOutOff + 8192 * (warp & 3);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if ((s == 0 ? it.n0 : it.n1) > 0) {
            const bool live = it.q0 + 128 * s + lane_row < it.Lq;  // rows beyond the valid length are written as zeros
            const uint32_t o_addr = tmem_lane + kColO + D * s;
            uint8_t* st_row = stage + 4096 * s + lane * 128;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t ra[16], rb[16];
              tmem_ld16(o_addr + 32 * h, ra);
              tmem_ld16(o_addr + 32 * h + 16, rb);
              tmem_ld_wait_for(ra);
              tmem_ld_wait_for(rb);
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                const uint32_t* r = (q4 < 2) ? ra + 8 * q4 : rb + 8 * (q4 - 2);
                uint4 w;
                w.x = pack2<kBF16>(__uint_as_float(r[0]), __uint_as_float(r[1]));
                w.y = pack2<kBF16>(__uint_as_float(r[2]), __uint_as_float(r[3]));
                w.z = pack2<kBF16>(__uint_as_float(r[4]), __uint_as_float(r[5]));
                w.w = pack2<kBF16>(__uint_as_float(r[6]), __uint_as_float(r[7]));
                if (!live) w = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(st_row + (((4 * h + q4) ^ (lane & 7)) << 4)) = w;
              }
            }
          }
        }
        if (it.n_max > 0) {
          // O has left TMEM: the next item's products may overwrite the accumulators
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(L::kOEmpty));
        }
        __syncwarp();
        const int sub_row = lane >> 3, ch = lane & 7;
        uint8_t* o_base = reinterpret_cast<uint8_t*>(p.o) +
                          2 * ((int64_t)it.bc * p.o_sb + (int64_t)it.h * p.o_sh +
                               (int64_t)(it.tq0 + it.q0 + 32 * (warp & 3) + sub_row) * p.o_st) + 16 * ch;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const bool has_o = (s == 0 ? it.n0 : it.n1) > 0;  // else the tile is entirely padding: zero rows
          // this lane's rows of the tile are sub_row, sub_row + 4, ...; row 4 i + sub_row may be written if 4 i < rows_left
          const int rows_left = it.row_lim - (it.q0 + 128 * s + 32 * (warp & 3) + sub_row);
          uint8_t* o_ptr = o_base + 2 * (int64_t)(128 * s) * p.o_st;
          const uint8_t* st_ptr = stage + 4096 * s + sub_row * 128;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            uint4 w = make_uint4(0, 0, 0, 0);
            // (4 i + sub_row) & 7 = sub_row for even i, sub_row + 4 for odd i
            if (has_o) w = *reinterpret_cast<const uint4*>(st_ptr + 512 * i + ((ch ^ ((sub_row + 4 * (i & 1)) & 7)) << 4));
            if (4 * i < rows_left) *reinterpret_cast<uint4*>(o_ptr) = w;
            o_ptr += 8 * p.o_st;
          }
        }
        __syncwarp();  // the patches are free again
      } else {
      // D = 128: room to stage one query tile at a time (32 rows x 256 bytes per warp).  Tile 0 goes through the
      // patch and out, then tile 1; the accumulators are handed back after the last TMEM load.  Rows leave
      // with sixteen lanes per 256-byte row; a lane writing its own row's columns as they come out of TMEM
      // touched 32 lines per store instruction, which the load/store unit takes one at a time (about 4000
      // clocks per item) and which held the hand-back up, since the loads were interleaved with those stores.
      uint8_t* stage = smem_gen + L::kOutOff + 8192 * (warp & 3);
      uint8_t* o_base = reinterpret_cast<uint8_t*>(p.o) +
                        2 * ((int64_t)it.bc * p.o_sb + (int64_t)it.h * p.o_sh +
                             (int64_t)(it.tq0 + it.q0 + 32 * (warp & 3) + (lane >> 4)) * p.o_st) + 16 * (lane & 15);
      const int last_tile = it.n1 > 0 ? 1 : 0;  // the last tile that has accumulators to read (n_max > 0 means n0 > 0 or n1 > 0)
#pragma unroll 1
      for (int s = 0; s < 2; ++s) {
        const bool has_o = (s == 0 ? it.n0 : it.n1) > 0;  // else the tile is entirely padding: zero rows
        if (has_o) {
          const bool live = it.q0 + 128 * s + lane_row < it.Lq;  // rows beyond the valid length are written as zeros
          const uint32_t o_addr = tmem_lane + kColO + D * s;
          uint8_t* st_row = stage + lane * 256;
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            uint32_t ra[16], rb[16];
            tmem_ld16(o_addr + 32 * h, ra);
            tmem_ld16(o_addr + 32 * h + 16, rb);
            tmem_ld_wait_for(ra);
            tmem_ld_wait_for(rb);
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              const uint32_t* r = (q4 < 2) ? ra + 8 * q4 : rb + 8 * (q4 - 2);
              uint4 w;
              w.x = pack2<kBF16>(__uint_as_float(r[0]), __uint_as_float(r[1]));
              w.y = pack2<kBF16>(__uint_as_float(r[2]), __uint_as_float(r[3]));
              w.z = pack2<kBF16>(__uint_as_float(r[4]), __uint_as_float(r[5]));
              w.w = pack2<kBF16>(__uint_as_float(r[6]), __uint_as_float(r[7]));
              if (!live) w = make_uint4(0, 0, 0, 0);
              // 16-byte chunk 4 h + q4 of the row, its low three bits swizzled by the row
              *reinterpret_cast<uint4*>(st_row + ((((4 * h + q4) & 8) | (((4 * h + q4) ^ lane) & 7)) << 4)) = w;
            }
          }
        }
        if (it.n_max > 0 && s == last_tile) {
          // O has left TMEM: the next item's products may overwrite the accumulators
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(L::kOEmpty));
        }
        __syncwarp();
        // this lane's rows of the tile are (lane >> 4), (lane >> 4) + 2, ...; row 2 i + (lane >> 4) may be written if 2 i < rows_left
        const int rows_left = it.row_lim - (it.q0 + 128 * s + 32 * (warp & 3) + (lane >> 4));
        uint8_t* o_ptr = o_base + 2 * (int64_t)(128 * s) * p.o_st;
        const int ch = lane & 15;
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
          const int r = 2 * i + (lane >> 4);
          uint4 w = make_uint4(0, 0, 0, 0);
          if (has_o) w = *reinterpret_cast<const uint4*>(stage + r * 256 + (((ch & 8) | ((ch ^ r) & 7)) << 4));
          if (2 * i < rows_left) *reinterpret_cast<uint4*>(o_ptr) = w;
          o_ptr += 4 * p.o_st;
        }
        __syncwarp();  // the patch is free again
      }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(L::kItemEmpty + islot));
    }
  } else if (warp >= kFwdSigmoidWarps) {
  // All four role warps (the idle one included) execute this one instruction: the release is an
  // operation of the whole group of four.
  setmaxnreg_dec<FwdRegs<D>::kRole>();
  if (warp == kFwdProducerWarp) {
    // ============================================================ item scheduler + TMA producer
    int tile = 0;        // key tiles loaded so far (all items): position in the stage ring
    int act = 0;         // items with work so far
    bool ok = true;
    for (int k = 0; ok; ++k) {
      const int slot = k & 1;
      ok = mbar_wait_warp(bar(L::kItemEmpty + slot), ((uint32_t)(k >> 1) & 1u) ^ 1u, abort_flag, kSiteBase + 31);
      if (!ok) break;
      int item = blockIdx.x;  // the first item needs no ticket
      if (lane == 0 && k > 0) {
        const unsigned int t = atomicAdd(p.ticket, 1u) + gridDim.x;
        item = t < (unsigned int)p.n_items ? (int)t : -1;
      }
      item = __shfl_sync(0xffffffffu, item, 0);
      FwdItem it = {};
      if (item >= 0) it = fwd_decode_item(p, item);
      if (lane == 0) {
        if (item >= 0) fwd_publish_item(item_ring + 16 * slot, item, it);
        else item_ring[16 * slot] = -1;
        mbar_arrive(bar(L::kItemFull + slot));  // (release: the record is visible to whoever sees the phase)
      }
      if (item < 0) break;
      if (it.n_max == 0) continue;

      // Q tiles of this item: the previous item's score products must have read theirs
      if (act > 0) ok = mbar_wait_warp(bar(L::kQEmpty), (uint32_t)(act - 1) & 1u, abort_flag, kSiteBase + 32);
      if (!ok) break;
      if (lane == 0) {
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if ((s == 0 ? it.n0 : it.n1) > 0) {
            mbar_expect_tx(bar(L::kQFull + s), kTileBytes);
#pragma unroll
            for (int c = 0; c < D / 64; ++c)
              tma_load_4d(smem_base + L::kQOff + s * kTileBytes + c * 16384, &q_map, bar(L::kQFull + s), c * 64, it.h,
                          it.tq0 + it.q0 + 128 * s, it.bc);
          }
        }
      }
      int st = tile % kStages;
      uint32_t ph = (uint32_t)(tile / kStages) & 1u;
      for (int j = 0; j < it.n_max && ok; ++j) {
        ok = mbar_wait_warp(bar(L::kKEmpty + st), ph ^ 1u, abort_flag, kSiteBase + 1);
        if (!ok) break;
        if (lane == 0) {
          mbar_expect_tx(bar(L::kKFull + st), kTileBytes);
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_4d(smem_base + L::kKOff + st * kTileBytes + c * 16384, &k_map, bar(L::kKFull + st), c * 64, it.h,
                        it.tk0 + j * kTileN, it.bc);
        }
        ok = mbar_wait_warp(bar(L::kVEmpty + st), ph ^ 1u, abort_flag, kSiteBase + 2);
        if (!ok) break;
        if (lane == 0) {
          mbar_expect_tx(bar(L::kVFull + st), kTileBytes);
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_4d(smem_base + L::kVOff + st * kTileBytes + c * 16384, &v_map, bar(L::kVFull + st), c * 64, it.h,
                        it.tk0 + j * kTileN, it.bc);
        }
        if (j * kTileN + kTileN > it.Lk) {
          // The tile straddles the valid key length.  P is zero for the padded keys, but 0 * NaN
          // is NaN inside the MMA, so whatever sits in the padded V rows must be cleared first.
          ok = mbar_wait_warp(bar(L::kVFull + st), ph, abort_flag, kSiteBase + 13);
          if (!ok) break;
          const int first_bad = it.Lk - j * kTileN;  // in [1, 127]
          uint8_t* vt = smem_gen + L::kVOff + st * kTileBytes;
          // each row is one 128-byte line per 64-column block; the swizzle only permutes within a line
          for (int i = lane; i < (kTileN - first_bad) * 8 * (D / 64); i += 32) {
            const int c = i / ((kTileN - first_bad) * 8);
            const int rem = i % ((kTileN - first_bad) * 8);
            const int r = first_bad + rem / 8;
            *reinterpret_cast<uint4*>(vt + c * 16384 + r * 128 + (rem % 8) * 16) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(L::kVFix + st));
        }
        if (++st == kStages) { st = 0; ph ^= 1u; }
      }
      tile += it.n_max;
      ++act;
    }
  }
  else if (warp == kFwdIssuerWarp) {
    // ============================================================ tcgen05 issuer 1: S = Q K^T
    // Two issuing warps (this one for the scores, the next for P V): an issuing warp's
    // instruction stream is one long dependent chain (waits, MMAs, commits), and a single warp
    // doing both products was what bounded the kernel.  All ring positions, stage numbers and
    // barrier parities are carried incrementally (no division, no modulo) and run on across
    // items; descriptors are a precomputed base plus a constant in the start-address field.
    const bool leader = elect_one();
    constexpr uint32_t idesc_qk = make_idesc(128, 128, kBF16, false, false);
    constexpr uint32_t kStageStep = kTileBytes >> 4;  // one smem stage, in descriptor address units
    // Q tile 0 and K stage 0: rows = M/N, the 64 contiguous elements = contraction
    const uint64_t q_desc0 = smem_desc_sw128(smem_base + L::kQOff, 16, 1024);
    const uint64_t k_desc0 = smem_desc_sw128(smem_base + L::kKOff, 16, 1024);
    const uint32_t q_lo = (uint32_t)q_desc0, k_lo = (uint32_t)k_desc0, hi = (uint32_t)(q_desc0 >> 32);
    FwdCursor c{0, 0, 0, 0u, 0, 0u, true};
    uint32_t q_par0 = 0u, q_par1 = 0u;  // parity of each Q tile's "full" barrier
    int total = 0;                 // jobs issued so far, saturating at kSBufs
    bool ok = true;
    for (int k = 0; ok; ++k) {
      FwdItem it;
      const int item = read_item(k, it);
      if (item < 0) break;
      if (it.n_max == 0) continue;
      const int n0 = it.n0, n1 = it.n1;
      const int n_jobs = n0 + n1;
      c.begin_item(n0);
      for (int n = 0; n < n_jobs && ok; ++n) {
        if (c.j == 0) ok = mbar_wait_warp(bar(L::kQFull + c.s), (c.s ? q_par1 : q_par0), abort_flag, kSiteBase + 3);
        if (c.fresh) ok = ok && mbar_wait_warp(bar(L::kKFull + c.st), c.ph, abort_flag, kSiteBase + 5);
        // the buffer still holds the probabilities of the job kSBufs earlier until their P V product is complete
        if (total >= kSBufs) ok = ok && mbar_wait_warp(bar(L::kPvDone + c.buf), c.bph ^ 1u, abort_flag, kSiteBase + 4);
        else ++total;
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t qa = q_lo + (uint32_t)c.s * kStageStep;
        const uint32_t ka = k_lo + (uint32_t)c.st * kStageStep;
        const uint32_t dst = tmem + kColS + 128u * (uint32_t)c.buf;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (uint32_t)(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
          mma_ss(leader, dst, make_desc(qa + off, hi), make_desc(ka + off, hi), idesc_qk, kk > 0);
        }
        mma_commit(leader, bar(L::kSFull + c.buf));
        // last job that reads K_j: hand the stage back to the producer
        if (c.s == 1 || c.j >= n1) mma_commit(leader, bar(L::kKEmpty + c.st));
        c.advance(n0, n1, kStages, kSBufs);
      }
      if (!ok) break;
      mma_commit(leader, bar(L::kQEmpty));  // the Q tiles may be overwritten once these products are complete
      if (n0 > 0) q_par0 ^= 1u;
      if (n1 > 0) q_par1 ^= 1u;
    }
  } else if (warp == kFwdIssuerWarp2) {
    // ============================================================ tcgen05 issuer 2: O_s += P V_j
    const bool leader = elect_one();
    constexpr uint32_t idesc_pv = make_idesc(128, D, kBF16, false, true);
    constexpr uint32_t kStageStep = kTileBytes >> 4;
    // V stage 0: rows = contraction, the 64 contiguous elements = N, next 64-column block 16 KB further
    const uint64_t v_desc0 = smem_desc_sw128(smem_base + L::kVOff, 16384, 1024);
    const uint32_t v_lo = (uint32_t)v_desc0, hi = (uint32_t)(v_desc0 >> 32);
    FwdCursor c{0, 0, 0, 0u, 0, 0u, true};
    uint32_t fix_par = 0u;  // bit st: parity of stage st's "padded V rows cleared" barrier
    int act = 0;            // items with work so far
    bool ok = true;
    for (int k = 0; ok; ++k) {
      FwdItem it;
      const int item = read_item(k, it);
      if (item < 0) break;
      if (it.n_max == 0) continue;
      const int n0 = it.n0, n1 = it.n1;
      const int n_jobs = n0 + n1;
      c.begin_item(n0);
      // the accumulators still hold the previous item's O until the sigmoid warps have read it
      if (act > 0) ok = mbar_wait_warp(bar(L::kOEmpty), (uint32_t)(act - 1) & 1u, abort_flag, kSiteBase + 33);
      for (int n = 0; n < n_jobs && ok; ++n) {
        if (c.fresh) {
          ok = mbar_wait_warp(bar(L::kVFull + c.st), c.ph, abort_flag, kSiteBase + 6);
          if (c.j * kTileN + kTileN > it.Lk) {  // padded V rows are being cleared by the producer warp
            ok = ok && mbar_wait_warp(bar(L::kVFix + c.st), (fix_par >> c.st) & 1u, abort_flag, kSiteBase + 14);
            fix_par ^= 1u << c.st;
          }
        }
        ok = ok && mbar_wait_warp(bar(L::kPFull + c.buf), c.bph, abort_flag, kSiteBase + 7);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t va = v_lo + (uint32_t)c.st * kStageStep;
        const uint32_t pa = tmem + kColS + 128u * (uint32_t)c.buf;
        const uint32_t dst = tmem + kColO + (uint32_t)(D * c.s);
        const uint32_t acc0 = c.j > 0 ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < kTileN / 16; ++kk) {
          // P of key columns [32g, 32g+32) sits, 16-bit packed, in buffer columns 32g + [0,16)
          mma_ts(leader, dst, pa + 32 * (kk >> 1) + 8 * (kk & 1), make_desc(va + kk * (2048 >> 4), hi), idesc_pv,
                 kk > 0 ? 1u : acc0);
        }
        mma_commit(leader, bar(L::kPvDone + c.buf));
        if (c.s == 1 || c.j >= n1) mma_commit(leader, bar(L::kVEmpty + c.st));
        c.advance(n0, n1, kStages, kSBufs);
      }
      if (!ok) break;
      mma_commit(leader, bar(L::kOFull));
      ++act;
    }
  }
  }  // role warps
  else {
    // ============================================================ sigmoid warps
    setmaxnreg_inc<FwdRegs<D>::kSigmoid>();
    const int cq = warp >> 2;                         // quarter of a job's key columns (16 warps per job) / of the head dimension in the epilogue
    const int lane_row = (warp & 3) * 32 + lane;      // TMEM lane == row within a query tile
    const uint32_t tmem_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const float c1 = p.scale * kLog2e;
    int buf = 0;          // 16 warps per job: S buffer of the next job
    uint32_t bph = 0u;    //                   and the parity of that buffer's barriers
    int jobs_base = 0;    // 8 warps per job: jobs of all earlier items, position of this item's first job in the S ring
    bool ok = true;

    for (int k = 0; ok; ++k) {
      const int islot = k & 1;
      ok = mbar_wait_warp(bar(L::kItemFull + islot), (uint32_t)(k >> 1) & 1u, abort_flag, kSiteBase + 30);
      if (!ok) break;
      const int item = item_ring[16 * islot];
      if (item < 0) break;
      int n0, n1, q0, Lk;
      float c0;
      const float* sm_row = nullptr;
      int sm_lim = 0;
      {
        const FwdItem it = fwd_load_item(item_ring + 16 * islot);
        n0 = it.n0;
        n1 = it.n1;
        q0 = it.q0;
        Lk = it.Lk;
        c0 = it.bias * kLog2e;
        if constexpr (kScoreMod) {
          sm_row = p.score_mod + (p.cu_k ? (int64_t)it.tk0 : (int64_t)it.b * p.Tk);
          sm_lim = it.key_lim;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(L::kItemEmpty + islot));  // the record is in registers
      // per query tile: largest visible key index of this thread's row, and the first key index at which a
      // chunk needs the element predicate (it reaches beyond the keys every row of the tile sees)
      int lim[2], mask_from[2];
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        lim[s] = Lk - 1;
        mask_from[s] = Lk;
        if (p.causal) {
          lim[s] = min(lim[s], q0 + 128 * s + lane_row);
          mask_from[s] = min(mask_from[s], q0 + 128 * s + 1);
        }
      }
      const int n_max = max(n0, n1);

      if constexpr (kJobWarps == 16) {
        // every warp works on every job, in the fixed order (0,0) (1,0) (0,1) (1,1) ... restricted to j < n_s
        // (loading the next job's scores under this job's arithmetic was measured much slower: the second
        // register buffer makes the compiler spill inside the loop)
        for (int j = 0; j < n_max && ok; ++j) {
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            if (j < (s == 0 ? n0 : n1)) {
              ok = ok && mbar_wait_warp(bar(L::kSFull + buf), bph, abort_flag, kSiteBase + 10 + s);
              if (ok) {
                tc_fence_after_sync();
                const uint32_t s_addr = tmem_lane + kColS + 128u * (uint32_t)buf + 32u * (uint32_t)cq;
                const int col0 = j * kTileN + 32 * cq;
                uint32_t r[32];
                tmem_ld32_sync(s_addr, r);
                // the predicate code exists only in the instantiation used by boundary chunks
                if (col0 + 32 > mask_from[s])
                  fwd_sigmoid_chunk<kBF16, kScoreMod, true, kAccurate>(s_addr, r, c1, c0, col0, lim[s], sm_row, sm_lim);
                else
                  fwd_sigmoid_chunk<kBF16, kScoreMod, false, kAccurate>(s_addr, r, c1, c0, col0, lim[s], sm_row, sm_lim);
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(L::kPFull + buf));  // one arrival per warp: 512 on one barrier would serialise
                if (++buf == kSBufs) { buf = 0; bph ^= 1u; }
              }
            }
          }
        }
      } else {
        // warps 0-7: jobs of query tile 0, warps 8-15: tile 1; each warp 64 key columns of its jobs.
        // Jobs are ordered by key tile, query tile 0 before 1: (0,0) (1,0) (0,1) (1,1) ... restricted to
        // j < n_s, and numbered on across items; job n uses score buffer n % kSBufs in phase n / kSBufs.
        // The two groups run on across items independently of each other, and a barrier wait only knows the
        // phase's parity, so a group must never ask for a job more than kSBufs positions after the last one
        // whose barrier it has seen.  Within and between items in which its tile has jobs that holds by
        // itself (n1 - n0 is 0 or 1, or n1 = 0: at most two foreign jobs in a row).  A group whose tile has
        // NO job in an item (a query tile beyond the valid length) therefore does not just skip the item: it
        // watches the barrier of every one of its jobs go by.
        const int s = warp >> 3;
        const int g = (warp >> 2) & 1;
        const int n_mine = s == 0 ? n0 : n1;
        if (n_mine == 0) {
          for (int n = jobs_base; n < jobs_base + n0 + n1 && ok; ++n)
            ok = mbar_wait_warp(bar(L::kSFull + n % kSBufs), (uint32_t)(n / kSBufs) & 1u, abort_flag, kSiteBase + 10 + s);
        }
        for (int j = 0; j < n_mine && ok; ++j) {
          const int n = jobs_base + (s == 0 ? j + min(j, n1) : j + min(j + 1, n0));
          const int jb = n % kSBufs;
          ok = mbar_wait_warp(bar(L::kSFull + jb), (uint32_t)(n / kSBufs) & 1u, abort_flag, kSiteBase + 10 + s);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t s_addr = tmem_lane + kColS + 128u * (uint32_t)jb + 64u * (uint32_t)g;
          const int col0 = j * kTileN + 64 * g;
          // two register buffers: the load of the second chunk is in flight while the first is computed
          uint32_t rbuf[2][32];
          tmem_ld(s_addr, rbuf[0]);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t(&r)[32] = rbuf[c];
            tmem_ld_wait_for(r);
            if (c == 0) tmem_ld(s_addr + 32, rbuf[1]);
            if (col0 + 32 * c + 32 > mask_from[s])
              fwd_sigmoid_chunk<kBF16, kScoreMod, true, kAccurate>(s_addr + 32 * c, r, c1, c0, col0 + 32 * c, lim[s], sm_row, sm_lim);
            else
              fwd_sigmoid_chunk<kBF16, kScoreMod, false, kAccurate>(s_addr + 32 * c, r, c1, c0, col0 + 32 * c, lim[s], sm_row, sm_lim);
          }
          tmem_st_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(L::kPFull + jb));  // one arrival per warp: 256 on one barrier would serialise
        }
        if (!ok) break;
        jobs_base += n0 + n1;
      }
      if (!ok) break;

      // the item's accumulators are the output warps' business; on to the next item
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kFwdIssuerWarp) {
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
