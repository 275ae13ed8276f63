// Forward kernel: O = sigmoid(scale * Q K^T + bias) V for one (batch, head, 256-query block)
// per CTA.
//
// Takes over the work of the reference's _fwd_dense_kernel
// (src/triton_sigmoid/sigmoid_triton_dense.py:23-154) and _fwd_padded_kernel
// (src/triton_sigmoid/sigmoid_triton_padded.py:24-171).
//
// Structure (sm_100a, 20 warps):
//   warps 0-7    sigmoid groups of query tile 0 (rows [q0, q0+128)): warps 0-3 take key columns
//                [0,64) of every score tile, warps 4-7 columns [64,128); one thread per row
//   warps 8-15   the same for query tile 1 (rows [q0+128, q0+256))
//   warp  16     TMA producer: Q tiles once, then K_j / V_j through a ring of smem stages
//   warp  17     tcgen05 issuer 1: S = Q_s K_j^T (smem x smem -> TMEM fp32); owns the TMEM allocation
//   warp  18     tcgen05 issuer 2: O_s += P V_j (TMEM x smem -> TMEM fp32)
//   warp  19     idle
// There is no row normaliser in sigmoid attention, so O simply accumulates in TMEM over the
// whole key loop.  The (query tile, key tile) jobs are processed in a fixed order through a
// small ring of S buffers in TMEM (3 when D = 64, 2 when D = 128): the issuer computes the
// scores of a later job while the sigmoid groups turn earlier ones into 16-bit P in place
// (each group writes P over the start of the columns it has just read) and signal the issuer.
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
  const float* bias;       // [B] or nullptr
  const float* score_mod;  // [B, Tk] or nullptr
  float scale;
  float bias_scalar;
  int B, H, Tq, Tk;
  int causal;
  int n_qblk;  // ceil(Tq / 256)
};

#ifndef SIG_FWD_CHUNK
#define SIG_FWD_CHUNK 32  // score columns per TMEM load of a sigmoid thread (32 measured faster than 16)
#endif
#ifndef SIG_FWD_HALVES
#define SIG_FWD_HALVES 2  // sigmoid warps per (query tile, lane quarter): 2 = each takes 64 of the 128 key columns
#endif
constexpr int kFwdHalves = SIG_FWD_HALVES;
constexpr int kFwdSigmoidWarps = 8 * kFwdHalves;
constexpr int kFwdProducerWarp = kFwdSigmoidWarps;
constexpr int kFwdIssuerWarp = kFwdSigmoidWarps + 1;   // S = Q K^T, owns the TMEM allocation
constexpr int kFwdIssuerWarp2 = kFwdSigmoidWarps + 2;  // O += P V
constexpr int kFwdThreads = (kFwdSigmoidWarps + 4) * 32;
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
  static constexpr int kBarOff = kVOff + kStages * kTileBytes;
  // barrier slots (8 bytes each)
  static constexpr int kQFull = 0;                    // [2]
  static constexpr int kKFull = kQFull + 2;           // [kStages]
  static constexpr int kKEmpty = kKFull + kStages;    // [kStages]
  static constexpr int kVFull = kKEmpty + kStages;    // [kStages]
  static constexpr int kVEmpty = kVFull + kStages;    // [kStages]
  static constexpr int kSFull = kVEmpty + kStages;    // [kSBufs]
  static constexpr int kPFull = kSFull + kSBufs;      // [kSBufs]
  static constexpr int kOFull = kPFull + kSBufs;      // [1]
  static constexpr int kVFix = kOFull + 1;            // [1] padded rows of the last V tile zeroed
  static constexpr int kPvDone = kVFix + 1;           // [kSBufs] P V product of the buffer's job complete
  static constexpr int kNumBars = kPvDone + kSBufs;
  static constexpr int kMiscOff = kBarOff + 8 * kNumBars;  // tmem base (u32), abort flag (int)
  static constexpr int kTotal = kMiscOff + 16;
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

// Turns 64 score columns of one TMEM lane (this thread's query row) into 16-bit probabilities,
// written back over the first 32 of those columns.  col0 = key index of the first column,
// lim = largest visible key index of this row (used only when kMask).
template <bool kBF16, bool kScoreMod, bool kMask>
__device__ __forceinline__ void fwd_sigmoid_half_tile(uint32_t s_addr, float c1, float c0, int col0, int lim,
                                                      const float* sm_row, int Tk) {
  // two register buffers: the load of the next chunk is in flight while one is computed
  constexpr int kCh = SIG_FWD_CHUNK;  // score columns per chunk
  constexpr int kNCh = 64 / kCh;
  uint32_t rbuf[2][kCh];
  tmem_ld(s_addr, rbuf[0]);
#pragma unroll
  for (int c = 0; c < kNCh; ++c) {
    uint32_t(&r)[kCh] = rbuf[c & 1];
    tmem_ld_wait_for(r);
    if (c + 1 < kNCh) tmem_ld(s_addr + (c + 1) * kCh, rbuf[(c + 1) & 1]);
    uint32_t pk[kCh / 2];
    float2 t[kCh / 2];
#pragma unroll
    for (int i = 0; i < kCh / 2; ++i) {
      t[i] = __ffma2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), make_float2(c1, c1),
                        make_float2(c0, c0));
    }
    if constexpr (kScoreMod) {
      // per-key additive bias: the same value for every lane (row), read through the read-only path
      const int cbase = col0 + c * kCh;
      if (cbase + kCh <= Tk && (reinterpret_cast<uintptr_t>(sm_row + cbase) & 15u) == 0) {
#pragma unroll
        for (int i = 0; i < kCh / 4; ++i) {
          const float4 m = __ldg(reinterpret_cast<const float4*>(sm_row + cbase) + i);
          t[2 * i] = __ffma2_rn(make_float2(m.x, m.y), make_float2(kLog2e, kLog2e), t[2 * i]);
          t[2 * i + 1] = __ffma2_rn(make_float2(m.z, m.w), make_float2(kLog2e, kLog2e), t[2 * i + 1]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < kCh / 2; ++i) {
          const int col = cbase + 2 * i;
          t[i].x = fmaf(col < Tk ? __ldg(sm_row + col) : 0.0f, kLog2e, t[i].x);
          t[i].y = fmaf(col + 1 < Tk ? __ldg(sm_row + col + 1) : 0.0f, kLog2e, t[i].y);
        }
      }
    }
    // Under the default bias every logit of a chunk is negative: then the sign handling (one
    // compare and one select per element) is skipped for the whole warp.
    if (!kMask && warp_all_negative(t)) {
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
          const int col = col0 + c * kCh + 2 * i;
          pr.x = (col <= lim) ? pr.x : 0.0f;
          pr.y = (col + 1 <= lim) ? pr.y : 0.0f;
        }
        pk[i] = pack2<kBF16>(pr.x, pr.y);
      }
    }
    tmem_st(s_addr + c * (kCh / 2), pk);
  }
}

template <int D, bool kBF16, bool kScoreMod>
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
  // D = 64: scores and P V are issued by two warps (the issue stream bounds the kernel); D = 128:
  // one warp issues both, in order - with only two S buffers the extra barrier hop costs more
  constexpr bool kSplitIssue = (D == 64);
  static_assert(kColO + 2 * D <= kTmemCols, "TMEM budget");

  extern __shared__ uint8_t smem_dyn[];
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
  const uint32_t bars = smem_base + L::kBarOff;
  auto bar = [&](int slot) -> uint32_t { return bars + 8u * slot; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---------------------------------------------------------------- work item
  const int qblk = p.causal ? (p.n_qblk - 1 - (int)blockIdx.x) : (int)blockIdx.x;  // heavy blocks first
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int q0 = qblk * kFwdBlockM;
  int Lq = p.Tq, Lk = p.Tk;
  if (p.lens_q) Lq = min(max(p.lens_q[b], 0), p.Tq);
  if (p.lens_k) Lk = min(max(p.lens_k[b], 0), p.Tk);

  // key-tile counts per query tile
  int n_kv[2];
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const int r0 = q0 + 128 * s;
    int kv_end = Lk;
    if (p.causal) kv_end = min(kv_end, r0 + 128);
    n_kv[s] = (r0 < Lq) ? (kv_end + kTileN - 1) / kTileN : 0;
  }
  const int n0 = n_kv[0], n1 = n_kv[1];
  const int n_max = max(n0, n1);
  // Jobs are ordered by key tile, query tile 0 before 1: (0,0) (1,0) (0,1) (1,1) ...
  // Index of job (s, j) in that order (only meaningful when j < n_kv[s]).
  auto job_index = [&](int s, int j) { return s == 0 ? j + min(j, n1) : j + min(j + 1, n0); };

  uint8_t* o_base = reinterpret_cast<uint8_t*>(p.o) + 2 * ((int64_t)b * p.o_sb + (int64_t)h * p.o_sh);

  if (n_max == 0) {
    // nothing visible to this block: the reference stores zeros for such rows
    constexpr int kChunksPerRow = D * 2 / 16;
    for (int i = threadIdx.x; i < kFwdBlockM * kChunksPerRow; i += kFwdThreads) {
      const int row = q0 + i / kChunksPerRow;
      if (row < p.Tq)
        *reinterpret_cast<uint4*>(o_base + 2 * (int64_t)row * p.o_st + 16 * (i % kChunksPerRow)) =
            make_uint4(0, 0, 0, 0);
    }
    return;
  }

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
      mbar_init(bar(L::kPFull + i), 4 * kFwdHalves);  // one arrival per sigmoid warp of the query tile
      mbar_init(bar(L::kPvDone + i), 1);
    }
    mbar_init(bar(L::kOFull), 1);
    mbar_init(bar(L::kVFix), 1);
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

  if (warp == kFwdProducerWarp) {
    // ============================================================ TMA producer
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        if (n_kv[s] > 0) {
          mbar_expect_tx(bar(L::kQFull + s), kTileBytes);
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_4d(smem_base + L::kQOff + s * kTileBytes + c * 16384, &q_map, bar(L::kQFull + s), c * 64, h,
                        q0 + 128 * s, b);
        }
      }
    }
    bool ok = true;
    for (int j = 0; j < n_max && ok; ++j) {
      const int st = j % kStages;
      const uint32_t ph = (j / kStages) & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kKEmpty + st), ph ^ 1, abort_flag, kSiteBase + 1));
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(bar(L::kKFull + st), kTileBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(smem_base + L::kKOff + st * kTileBytes + c * 16384, &k_map, bar(L::kKFull + st), c * 64, h,
                      j * kTileN, b);
      }
      ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kVEmpty + st), ph ^ 1, abort_flag, kSiteBase + 2));
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(bar(L::kVFull + st), kTileBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(smem_base + L::kVOff + st * kTileBytes + c * 16384, &v_map, bar(L::kVFull + st), c * 64, h,
                      j * kTileN, b);
      }
      if (j * kTileN + kTileN > Lk) {
        // The tile straddles the valid key length.  P is zero for the padded keys, but 0 * NaN
        // is NaN inside the MMA, so whatever sits in the padded V rows must be cleared first.
        ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kVFull + st), ph, abort_flag, kSiteBase + 13));
        if (!ok) break;
        const int first_bad = Lk - j * kTileN;  // in [1, 127]
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
        if (lane == 0) mbar_arrive(bar(L::kVFix));
      }
    }
  } else if (warp == kFwdIssuerWarp) {
    if constexpr (kSplitIssue) {
    // ============================================================ tcgen05 issuer 1: S = Q K^T
    // Two issuing warps (this one for the scores, the next for P V): an issuing warp's
    // instruction stream is one long dependent chain (waits, MMAs, commits), and a single warp
    // doing both products was what bounded the kernel.  All ring positions, stage numbers and
    // barrier parities are carried incrementally (no division, no modulo), and descriptors are a
    // precomputed base plus a constant in the start-address field.
    const bool leader = elect_one();
    constexpr uint32_t idesc_qk = make_idesc(128, 128, kBF16, false, false);
    constexpr uint32_t kStageStep = kTileBytes >> 4;  // one smem stage, in descriptor address units
    const int n_jobs = n0 + n1;
    // Q tile 0 and K stage 0: rows = M/N, the 64 contiguous elements = contraction
    const uint64_t q_desc0 = smem_desc_sw128(smem_base + L::kQOff, 16, 1024);
    const uint64_t k_desc0 = smem_desc_sw128(smem_base + L::kKOff, 16, 1024);
    const uint32_t q_lo = (uint32_t)q_desc0, k_lo = (uint32_t)k_desc0, hi = (uint32_t)(q_desc0 >> 32);
    FwdCursor c{(n0 > 0) ? 0 : 1, 0, 0, 0u, 0, 0u, true};
    bool ok = true;
    for (int n = 0; n < n_jobs && ok; ++n) {
      if (c.j == 0) ok = mbar_wait_warp(bar(L::kQFull + c.s), 0, abort_flag, kSiteBase + 3);
      if (c.fresh) ok = ok && mbar_wait_warp(bar(L::kKFull + c.st), c.ph, abort_flag, kSiteBase + 5);
      // the buffer still holds the probabilities of job n - kSBufs until their P V product is complete
      if (n >= kSBufs) ok = ok && mbar_wait_warp(bar(L::kPvDone + c.buf), c.bph ^ 1u, abort_flag, kSiteBase + 4);
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
    } else {
    // ============================================================ single tcgen05 issuer (D = 128)
    // This warp's instruction stream is one long dependent chain, so its length per job decides
    // how quickly finished probabilities turn into new scores: all ring positions, stage numbers
    // and barrier parities are carried incrementally (no division, no modulo), and descriptors
    // are a precomputed base plus a constant in the start-address field.
    {
      const bool leader = elect_one();
      constexpr uint32_t idesc_qk = make_idesc(128, 128, kBF16, false, false);
      constexpr uint32_t idesc_pv = make_idesc(128, D, kBF16, false, true);
      constexpr uint32_t kStageStep = kTileBytes >> 4;  // one smem stage, in descriptor address units
      const int n_jobs = n0 + n1;
      bool ok = true;
      // Q tile 0, K stage 0 (rows = M/N, the 64 contiguous elements = K) and V stage 0 (rows = K,
      // the 64 contiguous elements = N, next 64-column block 16 KB further)
      const uint64_t q_desc0 = smem_desc_sw128(smem_base + L::kQOff, 16, 1024);
      const uint64_t k_desc0 = smem_desc_sw128(smem_base + L::kKOff, 16, 1024);
      const uint64_t v_desc0 = smem_desc_sw128(smem_base + L::kVOff, 16384, 1024);
      const uint32_t q_lo = (uint32_t)q_desc0, q_hi = (uint32_t)(q_desc0 >> 32);
      const uint32_t k_lo = (uint32_t)k_desc0, k_hi = (uint32_t)(k_desc0 >> 32);
      const uint32_t v_lo = (uint32_t)v_desc0, v_hi = (uint32_t)(v_desc0 >> 32);

      FwdCursor cs{(n0 > 0) ? 0 : 1, 0, 0, 0u, 0, 0u, true};  // next scores to issue
      FwdCursor cp = cs;                                      // next P V product to issue

      // S[buf] = Q_s K_j^T
      auto issue_s = [&](const FwdCursor& c) {
        {
          if (c.j == 0) ok = ok && mbar_wait_warp(bar(L::kQFull + c.s), 0, abort_flag, kSiteBase + 3);
          if (c.fresh) ok = ok && mbar_wait_warp(bar(L::kKFull + c.st), c.ph, abort_flag, kSiteBase + 5);
        }
        if (!ok) return;
        const uint32_t qa = q_lo + (uint32_t)c.s * kStageStep;
        const uint32_t ka = k_lo + (uint32_t)c.st * kStageStep;
        const uint32_t dst = tmem + kColS + 128u * (uint32_t)c.buf;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (uint32_t)(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
          mma_ss(leader, dst, make_desc(qa + off, q_hi), make_desc(ka + off, k_hi), idesc_qk, kk > 0);
        }
        mma_commit(leader, bar(L::kSFull + c.buf));
        // last job that reads K_j: hand the stage back to the producer
        if (c.s == 1 || c.j >= n1) mma_commit(leader, bar(L::kKEmpty + c.st));
      };
      // O_s += P[buf] V_j
      auto issue_pv = [&](const FwdCursor& c) {
        {
          if (c.fresh) {
            ok = ok && mbar_wait_warp(bar(L::kVFull + c.st), c.ph, abort_flag, kSiteBase + 6);
            if (c.j * kTileN + kTileN > Lk)  // padded V rows are being cleared by the producer warp
              ok = ok && mbar_wait_warp(bar(L::kVFix), 0, abort_flag, kSiteBase + 14);
          }
          ok = ok && mbar_wait_warp(bar(L::kPFull + c.buf), c.bph, abort_flag, kSiteBase + 7);
        }
        if (!ok) return;
        tc_fence_after_sync();
        const uint32_t va = v_lo + (uint32_t)c.st * kStageStep;
        const uint32_t pa = tmem + kColS + 128u * (uint32_t)c.buf;
        const uint32_t dst = tmem + kColO + (uint32_t)(D * c.s);
        const uint32_t acc0 = c.j > 0 ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < kTileN / 16; ++kk) {
          // P of key columns [64g, 64g+64) sits, 16-bit packed, in buffer columns 64g + [0,32)
          mma_ts(leader, dst, pa + 64 * (kk >> 2) + 8 * (kk & 3), make_desc(va + kk * (2048 >> 4), v_hi), idesc_pv,
                 kk > 0 ? 1u : acc0);
        }
        if (c.s == 1 || c.j >= n1) mma_commit(leader, bar(L::kVEmpty + c.st));
      };

      int n_s = 0;
      for (; n_s < kSBufs && n_s < n_jobs && ok; ++n_s) {
        issue_s(cs);
        cs.advance(n0, n1, kStages, kSBufs);
      }
      for (int n = 0; n < n_jobs && ok; ++n) {
        issue_pv(cp);
        cp.advance(n0, n1, kStages, kSBufs);
        if (n_s < n_jobs && ok) {
          issue_s(cs);  // reuses the buffer the product above has just consumed
          cs.advance(n0, n1, kStages, kSBufs);
          ++n_s;
        }
      }
      if (ok) mma_commit(leader, bar(L::kOFull));
    }
    }
  } else if (warp == kFwdIssuerWarp2) {
    if constexpr (kSplitIssue) {
    // ============================================================ tcgen05 issuer 2: O_s += P V_j
    const bool leader = elect_one();
    constexpr uint32_t idesc_pv = make_idesc(128, D, kBF16, false, true);
    constexpr uint32_t kStageStep = kTileBytes >> 4;
    const int n_jobs = n0 + n1;
    // V stage 0: rows = contraction, the 64 contiguous elements = N, next 64-column block 16 KB further
    const uint64_t v_desc0 = smem_desc_sw128(smem_base + L::kVOff, 16384, 1024);
    const uint32_t v_lo = (uint32_t)v_desc0, hi = (uint32_t)(v_desc0 >> 32);
    FwdCursor c{(n0 > 0) ? 0 : 1, 0, 0, 0u, 0, 0u, true};
    bool ok = true;
    for (int n = 0; n < n_jobs && ok; ++n) {
      if (c.fresh) {
        ok = mbar_wait_warp(bar(L::kVFull + c.st), c.ph, abort_flag, kSiteBase + 6);
        if (c.j * kTileN + kTileN > Lk)  // padded V rows are being cleared by the producer warp
          ok = ok && mbar_wait_warp(bar(L::kVFix), 0, abort_flag, kSiteBase + 14);
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
        // P of key columns [64g, 64g+64) sits, 16-bit packed, in buffer columns 64g + [0,32)
        mma_ts(leader, dst, pa + 64 * (kk >> 2) + 8 * (kk & 3), make_desc(va + kk * (2048 >> 4), hi), idesc_pv,
               kk > 0 ? 1u : acc0);
      }
      mma_commit(leader, bar(L::kPvDone + c.buf));
      if (c.s == 1 || c.j >= n1) mma_commit(leader, bar(L::kVEmpty + c.st));
      c.advance(n0, n1, kStages, kSBufs);
    }
    if (ok) mma_commit(leader, bar(L::kOFull));
    }
  } else if (warp >= kFwdSigmoidWarps) {
    // idle warp
  } else {
    // ============================================================ sigmoid groups + epilogue
    const int s = warp / (4 * kFwdHalves);                // query tile
    const int g = kFwdHalves == 2 ? (warp >> 2) & 1 : 0;  // which half of the key columns (when split)
    constexpr int kColsMine = 128 / kFwdHalves;           // key columns per thread and job
    constexpr int kDMine = D / kFwdHalves;                // output columns per thread
    const int lane_row = (warp & 3) * 32 + lane;          // TMEM lane == row within the tile
    const int row = q0 + 128 * s + lane_row;              // query index
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const float c1 = p.scale * kLog2e;
    const float c0 = (p.bias ? p.bias[b] : p.bias_scalar) * kLog2e;
    const float* sm_row = kScoreMod ? (p.score_mod + (int64_t)b * p.Tk) : nullptr;
    uint8_t* o_row = o_base + 2 * (int64_t)row * p.o_st + g * D;  // this thread's output columns (16-bit)
    const int n_mine = n_kv[s];
    // largest visible key index for this row
    int lim = Lk - 1;
    if (p.causal) lim = min(lim, row);
    bool ok = true;

    for (int j = 0; j < n_mine; ++j) {
      const int n = job_index(s, j);
      const int buf = n % kSBufs;
      {
        ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kSFull + buf), (n / kSBufs) & 1, abort_flag, kSiteBase + 10 + s));
      }
      if (!ok) break;
      tc_fence_after_sync();
#pragma unroll
      for (int hh = 0; hh < kColsMine / 64; ++hh) {
        const uint32_t s_addr = tmem + lane_addr + kColS + 128 * buf + 64 * (g + hh);
        const int col0 = j * kTileN + 64 * (g + hh);
        const bool need_mask = (col0 + 64 > Lk) || (p.causal && col0 + 63 > q0 + 128 * s);
        // the predicate code exists only in the instantiation used by boundary tiles
        if (need_mask)
          fwd_sigmoid_half_tile<kBF16, kScoreMod, true>(s_addr, c1, c0, col0, lim, sm_row, p.Tk);
        else
          fwd_sigmoid_half_tile<kBF16, kScoreMod, false>(s_addr, c1, c0, col0, lim, sm_row, p.Tk);
      }
      {
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(L::kPFull + buf));  // 256 arrivals on one barrier would serialise
      }
    }

    if (n_mine == 0) {
      // this tile is entirely padding (or beyond Tq): zero rows
      if (row < p.Tq) {
#pragma unroll
        for (int c = 0; c < kDMine / 8; ++c) *reinterpret_cast<uint4*>(o_row + 16 * c) = make_uint4(0, 0, 0, 0);
      }
    } else if (ok) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kOFull), 0, abort_flag, kSiteBase + 12));
      if (ok) {
        tc_fence_after_sync();
        const uint32_t o_addr = tmem + lane_addr + kColO + D * s + g * kDMine;
        const bool live = row < Lq;
#pragma unroll
        for (int c = 0; c < kDMine / 32; ++c) {
          uint32_t r[32];
          tmem_ld32_sync(o_addr + c * 32, r);
          if (row < p.Tq) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 w;
              w.x = pack2<kBF16>(__uint_as_float(r[8 * q4 + 0]), __uint_as_float(r[8 * q4 + 1]));
              w.y = pack2<kBF16>(__uint_as_float(r[8 * q4 + 2]), __uint_as_float(r[8 * q4 + 3]));
              w.z = pack2<kBF16>(__uint_as_float(r[8 * q4 + 4]), __uint_as_float(r[8 * q4 + 5]));
              w.w = pack2<kBF16>(__uint_as_float(r[8 * q4 + 6]), __uint_as_float(r[8 * q4 + 7]));
              if (!live) w = make_uint4(0, 0, 0, 0);
              *reinterpret_cast<uint4*>(o_row + 64 * c + 16 * q4) = w;
            }
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kFwdIssuerWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace sigattn
