// Forward kernel: O = sigmoid(scale * Q K^T + bias) V for one (batch, head, 256-query block)
// per CTA.
//
// Takes over the work of the reference's _fwd_dense_kernel
// (src/triton_sigmoid/sigmoid_triton_dense.py:23-154) and _fwd_padded_kernel
// (src/triton_sigmoid/sigmoid_triton_padded.py:24-171).
//
// Structure (sm_100a):
//   warps 0-3   sigmoid group 0: owns query rows [q0, q0+128)      (one thread per row)
//   warps 4-7   sigmoid group 1: owns query rows [q0+128, q0+256)
//   warp  8     TMA producer: Q tiles once, then K_j / V_j through a ring of smem stages
//   warp  9     tcgen05 issuer: S_s = Q_s K_j^T (smem x smem -> TMEM fp32) and
//               O_s += P_s V_j (TMEM x smem -> TMEM fp32); also owns the TMEM allocation
//   warps 10-11 idle (pad the CTA to three warpgroups)
// There is no row normaliser in sigmoid attention, so O simply accumulates in TMEM over the
// whole key loop; the sigmoid groups turn S into 16-bit P in place (P aliases the first 64
// columns of S) and signal the issuer.  The two query tiles ping-pong so that tensor-core
// work for one overlaps the sigmoid of the other.
//
// Masking: key tiles beyond the causal diagonal or the valid key length are skipped
// entirely; tiles that straddle either boundary apply an element predicate.
#pragma once

#include "ptx.cuh"

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

constexpr int kFwdThreads = 384;
constexpr int kFwdBlockM = 256;  // query rows per CTA (two 128-row tiles)
constexpr int kTileN = 128;      // key rows per step
constexpr float kLog2e = 1.4426950408889634f;

template <int D>
struct FwdSmem {
  static constexpr int kStages = (D == 64) ? 4 : 2;
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
  static constexpr int kSFull = kVEmpty + kStages;    // [2]
  static constexpr int kPFull = kSFull + 2;           // [2]
  static constexpr int kOFull = kPFull + 2;           // [1]
  static constexpr int kVFix = kOFull + 1;            // [1] padded rows of the last V tile zeroed
  static constexpr int kNumBars = kVFix + 1;
  static constexpr int kMiscOff = kBarOff + 8 * kNumBars;  // tmem base (u32), abort flag (int)
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynBytes = kTotal + 1024;  // slack to align the base to 1024 bytes
};

// sigmoid(x) with x given in the base-2 domain (t = x * log2(e)).
// e = 2^-|t| in (0,1] (one MUFU op); sigmoid = (t < 0 ? e : 1) / (1 + e).  This keeps RELATIVE
// accuracy for strongly negative logits (the default bias is -log(T), so a typical probability
// is ~1/T), which 0.5 + 0.5 tanh(x/2) does not.  1/(1+e) on [0,1] is a minimax polynomial on
// the FMA pipe instead of a second MUFU op: the MUFU unit (16 results / clock / SM) is what
// bounds this kernel.  Maximum relative error of the polynomial: 5.1e-5 (degree 5, used for
// fp16, whose own rounding is 4.9e-4) and 3.0e-4 (degree 4, used for bf16, rounding 3.9e-3).
template <bool kBF16>
__device__ __forceinline__ float2 rcp1p_poly(float2 e) {
  float2 r;
  if constexpr (kBF16) {
    r = make_float2(0.1522425264120102f, 0.1522425264120102f);
    r = __ffma2_rn(r, e, make_float2(-0.5328524708747864f, -0.5328524708747864f));
    r = __ffma2_rn(r, e, make_float2(0.8658902645111084f, 0.8658902645111084f));
    r = __ffma2_rn(r, e, make_float2(-0.9848342537879944f, -0.9848342537879944f));
    r = __ffma2_rn(r, e, make_float2(0.9997026324272156f, 0.9997026324272156f));
  } else {
    r = make_float2(-0.1044827550649643f, -0.1044827550649643f);
    r = __ffma2_rn(r, e, make_float2(0.41793352365493774f, 0.41793352365493774f));
    r = __ffma2_rn(r, e, make_float2(-0.7705690264701843f, -0.7705690264701843f));
    r = __ffma2_rn(r, e, make_float2(0.9534193277359009f, 0.9534193277359009f));
    r = __ffma2_rn(r, e, make_float2(-0.9962754845619202f, -0.9962754845619202f));
    r = __ffma2_rn(r, e, make_float2(0.9999489784240723f, 0.9999489784240723f));
  }
  return r;
}

// Two sigmoids at once; t holds the logits times log2(e).
template <bool kBF16>
__device__ __forceinline__ float2 sigmoid2_from_log2(float2 t) {
  float2 e = make_float2(ex2_approx(-fabsf(t.x)), ex2_approx(-fabsf(t.y)));
  const float2 r = rcp1p_poly<kBF16>(e);
  e.x = t.x < 0.0f ? e.x : 1.0f;
  e.y = t.y < 0.0f ? e.y : 1.0f;
  return __fmul2_rn(e, r);
}

template <int D, bool kBF16, bool kScoreMod>
__global__ void __launch_bounds__(kFwdThreads, 1)
sigattn_fwd_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                   const __grid_constant__ CUtensorMap v_map, const FwdParams p) {
  using L = FwdSmem<D>;
  constexpr int kStages = L::kStages;
  constexpr int kTileBytes = L::kTileBytes;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0;    // S_s at kColS + 128 s (P_s aliases its first 64 columns)
  constexpr uint32_t kColO = 256;  // O_s at kColO + D s
  constexpr int kSiteBase = 0x10000;

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
  const int n_max = max(n_kv[0], n_kv[1]);

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
    mbar_init(bar(L::kSFull + 0), 1);
    mbar_init(bar(L::kSFull + 1), 1);
    mbar_init(bar(L::kPFull + 0), 128);
    mbar_init(bar(L::kPFull + 1), 128);
    mbar_init(bar(L::kOFull), 1);
    mbar_init(bar(L::kVFix), 1);
    fence_mbar_init();
  }
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&q_map);
    tma_prefetch_desc(&k_map);
    tma_prefetch_desc(&v_map);
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp == 8) {
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
  } else if (warp == 9) {
    // ============================================================ tcgen05 issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(128, 128, kBF16, false, false);
      constexpr uint32_t idesc_pv = make_idesc(128, D, kBF16, false, true);
      auto issue_s = [&](int s, int st) {
        const uint32_t qa = smem_base + L::kQOff + s * kTileBytes;
        const uint32_t ka = smem_base + L::kKOff + st * kTileBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          mma_ss(tmem + kColS + 128 * s, smem_desc_sw128(qa + off, 16, 1024), smem_desc_sw128(ka + off, 16, 1024),
                 idesc_qk, kk > 0);
        }
      };
      auto issue_pv = [&](int s, int st, bool first) {
        const uint32_t va = smem_base + L::kVOff + st * kTileBytes;
#pragma unroll
        for (int kk = 0; kk < kTileN / 16; ++kk) {
          mma_ts(tmem + kColO + D * s, tmem + kColS + 128 * s + kk * 8, smem_desc_sw128(va + kk * 2048, 16384, 1024),
                 idesc_pv, (!first || kk > 0) ? 1u : 0u);
        }
      };
      bool ok = true;
      if (n_kv[0] > 0) ok = ok && mbar_wait(bar(L::kQFull + 0), 0, abort_flag, kSiteBase + 3);
      if (n_kv[1] > 0) ok = ok && mbar_wait(bar(L::kQFull + 1), 0, abort_flag, kSiteBase + 4);
      ok = ok && mbar_wait(bar(L::kKFull + 0), 0, abort_flag, kSiteBase + 5);
      if (ok) {
        if (n_kv[0] > 0) { issue_s(0, 0); mma_commit(bar(L::kSFull + 0)); }
        if (n_kv[1] > 0) { issue_s(1, 0); mma_commit(bar(L::kSFull + 1)); }
        mma_commit(bar(L::kKEmpty + 0));
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int st = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        const int st_n = (j + 1) % kStages;
        const uint32_t ph_n = ((j + 1) / kStages) & 1;
        ok = mbar_wait(bar(L::kVFull + st), ph, abort_flag, kSiteBase + 6);
        if (!ok) break;
        if (j * kTileN + kTileN > Lk) {  // padded V rows are being cleared by the producer warp
          ok = mbar_wait(bar(L::kVFix), 0, abort_flag, kSiteBase + 14);
          if (!ok) break;
        }
        if (j < n_kv[0]) {
          ok = mbar_wait(bar(L::kPFull + 0), j & 1, abort_flag, kSiteBase + 7);
          if (!ok) break;
          tc_fence_after_sync();
          issue_pv(0, st, j == 0);
        }
        if (j + 1 < n_max) {
          ok = mbar_wait(bar(L::kKFull + st_n), ph_n, abort_flag, kSiteBase + 8);
          if (!ok) break;
        }
        if (j + 1 < n_kv[0]) { issue_s(0, st_n); mma_commit(bar(L::kSFull + 0)); }
        if (j < n_kv[1]) {
          ok = mbar_wait(bar(L::kPFull + 1), j & 1, abort_flag, kSiteBase + 9);
          if (!ok) break;
          tc_fence_after_sync();
          issue_pv(1, st, j == 0);
        }
        mma_commit(bar(L::kVEmpty + st));
        if (j + 1 < n_kv[1]) { issue_s(1, st_n); mma_commit(bar(L::kSFull + 1)); }
        if (j + 1 < n_max) mma_commit(bar(L::kKEmpty + st_n));
      }
      if (ok) mma_commit(bar(L::kOFull));
    }
  } else if (warp < 8) {
    // ============================================================ sigmoid groups + epilogue
    const int s = warp >> 2;
    const int lane_row = (warp & 3) * 32 + lane;          // TMEM lane == row within the tile
    const int row = q0 + 128 * s + lane_row;              // query index
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem + lane_addr + kColS + 128 * s;
    const uint32_t o_addr = tmem + lane_addr + kColO + D * s;
    const float c1 = p.scale * kLog2e;
    const float c0 = (p.bias ? p.bias[b] : p.bias_scalar) * kLog2e;
    const float* sm_row = kScoreMod ? (p.score_mod + (int64_t)b * p.Tk) : nullptr;
    uint8_t* o_row = o_base + 2 * (int64_t)row * p.o_st;
    const int n_mine = n_kv[s];
    bool ok = true;

    for (int j = 0; j < n_mine; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kSFull + s), j & 1, abort_flag, kSiteBase + 10 + s));
      if (!ok) break;
      tc_fence_after_sync();
      const int col0 = j * kTileN;
      // largest visible key index for this row
      int lim = Lk - 1;
      if (p.causal) lim = min(lim, row);
      const bool need_mask = (col0 + kTileN > Lk) || (p.causal && col0 + kTileN - 1 > q0 + 128 * s);
      // two register buffers: the load of chunk c+1 is in flight while chunk c is computed
      uint32_t rbuf[2][32];
      tmem_ld32(s_addr, rbuf[0]);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t(&r)[32] = rbuf[c & 1];
        tmem_ld_wait_for(r);
        if (c + 1 < 4) tmem_ld32(s_addr + (c + 1) * 32, rbuf[(c + 1) & 1]);
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float2 t = __ffma2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])),
                                make_float2(c1, c1), make_float2(c0, c0));
          const int col = col0 + c * 32 + 2 * i;
          if constexpr (kScoreMod) {
            t.x = fmaf(col < p.Tk ? __ldg(sm_row + col) : 0.0f, kLog2e, t.x);
            t.y = fmaf(col + 1 < p.Tk ? __ldg(sm_row + col + 1) : 0.0f, kLog2e, t.y);
          }
          float2 pr = sigmoid2_from_log2<kBF16>(t);
          if (need_mask) {
            pr.x = (col <= lim) ? pr.x : 0.0f;
            pr.y = (col + 1 <= lim) ? pr.y : 0.0f;
          }
          pk[i] = pack2<kBF16>(pr.x, pr.y);
        }
        tmem_st16(s_addr + c * 16, pk);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(bar(L::kPFull + s));
    }

    if (n_mine == 0) {
      // this tile is entirely padding (or beyond Tq): zero rows
      if (row < p.Tq) {
#pragma unroll
        for (int c = 0; c < D * 2 / 16; ++c) *reinterpret_cast<uint4*>(o_row + 16 * c) = make_uint4(0, 0, 0, 0);
      }
    } else if (ok) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kOFull), 0, abort_flag, kSiteBase + 12));
      if (ok) {
        tc_fence_after_sync();
        const bool live = row < Lq;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld32_sync(o_addr + c * 32, r);
          if (row < p.Tq) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 w;
              w.x = pack2<kBF16>(__uint_as_float(r[8 * g + 0]), __uint_as_float(r[8 * g + 1]));
              w.y = pack2<kBF16>(__uint_as_float(r[8 * g + 2]), __uint_as_float(r[8 * g + 3]));
              w.z = pack2<kBF16>(__uint_as_float(r[8 * g + 4]), __uint_as_float(r[8 * g + 5]));
              w.w = pack2<kBF16>(__uint_as_float(r[8 * g + 6]), __uint_as_float(r[8 * g + 7]));
              if (!live) w = make_uint4(0, 0, 0, 0);
              *reinterpret_cast<uint4*>(o_row + 64 * c + 16 * g) = w;
            }
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace sigattn
