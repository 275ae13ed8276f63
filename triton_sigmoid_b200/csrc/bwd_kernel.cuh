// Backward kernel: one CTA owns one (batch, head, 128-key tile), keeps K_j and V_j in shared
// memory and dK_j, dV_j in TMEM, and streams the query tiles Q_i, dO_i past them.
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
//   dQ_i  = dS K_j              (smem x smem -> TMEM), then added into an fp32 accumulator
//                                in global memory with vector reductions
//
// Warp roles (448 threads):
//   warps 0-3   compute group 0: query columns [0,64) of the tile, one key row per thread
//   warps 4-7   compute group 1: query columns [64,128)
//   warps 8-11  dQ drain: TMEM -> red.global.add.f32 (one query row per thread)
//   warp  12    TMA producer
//   warp  13    tcgen05 issuer, owns the TMEM allocation
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
  const float* bias;
  const float* score_mod;
  float scale;
  float bias_scalar;
  int B, H, Tq, Tk;
  int causal;
  int n_kvblk;
};

constexpr int kBwdThreads = 448;
constexpr int kBwdTileKV = 128;
constexpr int kBwdTileQ = 128;

template <int D>
struct BwdSmem {
  static constexpr int kStages = 2;
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kKOff + kTileBytes;
  static constexpr int kQOff = kVOff + kTileBytes;
  static constexpr int kDoOff = kQOff + kStages * kTileBytes;
  static constexpr int kDsOff = kDoOff + kStages * kTileBytes;
  static constexpr int kDsBytes = 128 * 128 * 2;
  static constexpr int kBarOff = kDsOff + kDsBytes;
  static constexpr int kKvFull = 0;
  static constexpr int kQFull = 1;                    // [2]
  static constexpr int kQEmpty = kQFull + kStages;    // [2]
  static constexpr int kDoFull = kQEmpty + kStages;   // [2]
  static constexpr int kDoEmpty = kDoFull + kStages;  // [2]
  static constexpr int kSFull = kDoEmpty + kStages;
  static constexpr int kDpFull = kSFull + 1;
  static constexpr int kPReady = kDpFull + 1;
  static constexpr int kDsReady = kPReady + 1;
  static constexpr int kDqFull = kDsReady + 1;
  static constexpr int kDqEmpty = kDqFull + 1;
  static constexpr int kDkvFull = kDqEmpty + 1;
  static constexpr int kKvFix = kDkvFull + 1;   // padded rows of K_j zeroed
  static constexpr int kQdoFix = kKvFix + 1;    // padded rows of the last Q_i / dO_i zeroed
  static constexpr int kNumBars = kQdoFix + 1;
  static constexpr int kMiscOff = kBarOff + 8 * kNumBars;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynBytes = kTotal + 1024;
};

template <int D, bool kBF16>
__global__ void __launch_bounds__(kBwdThreads, 1)
sigattn_bwd_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                   const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap do_map,
                   const BwdParams p) {
  using L = BwdSmem<D>;
  constexpr int kTileBytes = L::kTileBytes;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0;                      // S^T, 128 fp32 columns; P^T (16-bit) in columns 64g + [0,32)
  constexpr uint32_t kColDp = 128;                   // dP^T; dS^T (16-bit) in columns 64g + [0,32)
  constexpr uint32_t kColDv = 256;
  constexpr uint32_t kColDk = 256 + D;
  constexpr bool kDqAliased = (D == 128);            // no room left: dQ reuses the dP^T columns
  constexpr uint32_t kColDq = kDqAliased ? kColDp : 384;
  constexpr int kSiteBase = 0x20000;

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
  const int j = blockIdx.x;  // key tile
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int kv0 = j * kBwdTileKV;
  int Lq = p.Tq, Lk = p.Tk;
  if (p.lens_q) Lq = min(max(p.lens_q[b], 0), p.Tq);
  if (p.lens_k) Lk = min(max(p.lens_k[b], 0), p.Tk);
  const int i_end = (Lq + kBwdTileQ - 1) / kBwdTileQ;
  const int i_begin = p.causal ? j : 0;  // query tiles that can see this key tile (top-left aligned)
  const int n_q = (kv0 < Lk) ? max(i_end - i_begin, 0) : 0;

  uint8_t* dk_base = reinterpret_cast<uint8_t*>(p.dk) + 2 * ((int64_t)b * p.dk_sb + (int64_t)h * p.dk_sh);
  uint8_t* dv_base = reinterpret_cast<uint8_t*>(p.dv) + 2 * ((int64_t)b * p.dv_sb + (int64_t)h * p.dv_sh);

  if (n_q == 0) {
    constexpr int kChunksPerRow = D * 2 / 16;
    for (int i = threadIdx.x; i < kBwdTileKV * kChunksPerRow; i += kBwdThreads) {
      const int row = kv0 + i / kChunksPerRow;
      if (row < p.Tk) {
        *reinterpret_cast<uint4*>(dk_base + 2 * (int64_t)row * p.dk_st + 16 * (i % kChunksPerRow)) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(dv_base + 2 * (int64_t)row * p.dv_st + 16 * (i % kChunksPerRow)) = make_uint4(0, 0, 0, 0);
      }
    }
    return;
  }

  // a kernel of this library already gave up on a wait: do not pile more work on a sick device
  if (*reinterpret_cast<volatile int*>(&g_status_word) != 0) return;

  // ---------------------------------------------------------------- setup
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar(L::kKvFull), 1);
    for (int i = 0; i < L::kStages; ++i) {
      mbar_init(bar(L::kQFull + i), 1);
      mbar_init(bar(L::kQEmpty + i), 1);
      mbar_init(bar(L::kDoFull + i), 1);
      mbar_init(bar(L::kDoEmpty + i), 1);
    }
    mbar_init(bar(L::kSFull), 1);
    mbar_init(bar(L::kDpFull), 1);
    mbar_init(bar(L::kPReady), 256);
    mbar_init(bar(L::kDsReady), 256);
    mbar_init(bar(L::kDqFull), 1);
    mbar_init(bar(L::kDqEmpty), 128);
    mbar_init(bar(L::kDkvFull), 1);
    mbar_init(bar(L::kKvFix), 1);
    mbar_init(bar(L::kQdoFix), 1);
    fence_mbar_init();
  }
  if (warp == 12 && lane == 0) {
    tma_prefetch_desc(&q_map);
    tma_prefetch_desc(&k_map);
    tma_prefetch_desc(&v_map);
    tma_prefetch_desc(&do_map);
  }
  if (warp == 13) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp == 12) {
    // ============================================================ TMA producer
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
    if (lane == 0) {
      mbar_expect_tx(bar(L::kKvFull), 2 * kTileBytes);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_4d(smem_base + L::kKOff + c * 16384, &k_map, bar(L::kKvFull), c * 64, h, kv0, b);
        tma_load_4d(smem_base + L::kVOff + c * 16384, &v_map, bar(L::kKvFull), c * 64, h, kv0, b);
      }
    }
    bool ok = true;
    if (kv0 + kBwdTileKV > Lk) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kKvFull), 0, abort_flag, kSiteBase + 17));
      if (ok) {
        zero_rows(smem_gen + L::kKOff, Lk - kv0);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(L::kKvFix));
      }
    }
    for (int t = 0; t < n_q && ok; ++t) {
      const int st = t & 1;
      const uint32_t ph = (t >> 1) & 1;
      const int qrow = (i_begin + t) * kBwdTileQ;
      ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kQEmpty + st), ph ^ 1, abort_flag, kSiteBase + 1));
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(bar(L::kQFull + st), kTileBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(smem_base + L::kQOff + st * kTileBytes + c * 16384, &q_map, bar(L::kQFull + st), c * 64, h, qrow, b);
      }
      ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kDoEmpty + st), ph ^ 1, abort_flag, kSiteBase + 2));
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(bar(L::kDoFull + st), kTileBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(smem_base + L::kDoOff + st * kTileBytes + c * 16384, &do_map, bar(L::kDoFull + st), c * 64, h, qrow, b);
      }
      if (qrow + kBwdTileQ > Lq) {  // only the last query tile can straddle Lq
        ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kQFull + st), ph, abort_flag, kSiteBase + 18));
        ok = ok && __all_sync(0xffffffffu, mbar_wait(bar(L::kDoFull + st), ph, abort_flag, kSiteBase + 19));
        if (!ok) break;
        zero_rows(smem_gen + L::kQOff + st * kTileBytes, Lq - qrow);
        zero_rows(smem_gen + L::kDoOff + st * kTileBytes, Lq - qrow);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(L::kQdoFix));
      }
    }
  } else if (warp == 13) {
    // ============================================================ tcgen05 issuer
    {
      const bool leader = elect_one();
      constexpr uint32_t idesc_st = make_idesc(128, 128, kBF16, false, false);  // S^T, dP^T
      constexpr uint32_t idesc_acc = make_idesc(128, D, kBF16, false, true);    // dV, dK: A in TMEM, B rows = contraction
      constexpr uint32_t idesc_dq = make_idesc(128, D, kBF16, true, true);      // dQ: both operands row = contraction
      const uint32_t k_s = smem_base + L::kKOff;
      const uint32_t v_s = smem_base + L::kVOff;
      const uint32_t ds_s = smem_base + L::kDsOff;
      // descriptor bases; per-MMA descriptors differ only in the start-address field (>> 4)
      const uint64_t k_km = smem_desc_sw128(k_s, 16, 1024);        // K_j, rows = M
      const uint64_t v_km = smem_desc_sw128(v_s, 16, 1024);        // V_j, rows = M
      const uint64_t k_mn = smem_desc_sw128(k_s, 16384, 1024);     // K_j, rows = contraction
      const uint64_t ds_mn = smem_desc_sw128(ds_s, 16384, 1024);   // dS^T, rows = contraction
      const uint64_t q_km0 = smem_desc_sw128(smem_base + L::kQOff, 16, 1024);
      const uint64_t do_km0 = smem_desc_sw128(smem_base + L::kDoOff, 16, 1024);
      const uint64_t q_mn0 = smem_desc_sw128(smem_base + L::kQOff, 16384, 1024);
      const uint64_t do_mn0 = smem_desc_sw128(smem_base + L::kDoOff, 16384, 1024);
      constexpr uint64_t kStageStep = (uint64_t)(kTileBytes >> 4);
      // C[key, query] = A[key, :] . B[query, :] over the head dimension
      auto issue_kmajor = [&](uint32_t dcol, uint64_t a_d, uint64_t b_d) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t off = (uint64_t)(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
          mma_ss(leader, tmem + dcol, a_d + off, b_d + off, idesc_st, kk > 0);
        }
      };
      // acc[key, d] += A^T[key, query] (TMEM, 16-bit) . B[query, d] (smem tile of query rows)
      auto issue_acc = [&](uint32_t dcol, uint32_t acol, uint64_t b_d, bool first) {
        const uint32_t acc0 = first ? 0u : 1u;
#pragma unroll
        for (int kk = 0; kk < kBwdTileQ / 16; ++kk) {
          mma_ts(leader, tmem + dcol, tmem + acol + 64 * (kk >> 2) + 8 * (kk & 3), b_d + (uint64_t)(kk * (2048 >> 4)), idesc_acc,
                 kk > 0 ? 1u : acc0);
        }
      };
      auto ragged_q = [&](int t) { return (i_begin + t) * kBwdTileQ + kBwdTileQ > Lq; };
      bool ok = mbar_wait_warp(bar(L::kKvFull), 0, abort_flag, kSiteBase + 3);
      if (kv0 + kBwdTileKV > Lk) ok = ok && mbar_wait_warp(bar(L::kKvFix), 0, abort_flag, kSiteBase + 20);
      ok = ok && mbar_wait_warp(bar(L::kQFull + 0), 0, abort_flag, kSiteBase + 4);
      if (ragged_q(0)) ok = ok && mbar_wait_warp(bar(L::kQdoFix), 0, abort_flag, kSiteBase + 21);
      if (ok) {
        issue_kmajor(kColS, k_km, q_km0);
        mma_commit(leader, bar(L::kSFull));
      }
      ok = ok && mbar_wait_warp(bar(L::kDoFull + 0), 0, abort_flag, kSiteBase + 5);
      if (ok) {
        issue_kmajor(kColDp, v_km, do_km0);
        mma_commit(leader, bar(L::kDpFull));
      }
      for (int t = 0; t < n_q && ok; ++t) {
        const int st = t & 1;
        const uint64_t q_mn = q_mn0 + st * kStageStep;
        const uint64_t do_mn = do_mn0 + st * kStageStep;
        const int st_n = st ^ 1;
        const uint32_t ph_n = ((t + 1) >> 1) & 1;
        // dV += P^T dO
        ok = mbar_wait_warp(bar(L::kPReady), t & 1, abort_flag, kSiteBase + 6);
        if (!ok) break;
        tc_fence_after_sync();
        issue_acc(kColDv, kColS, do_mn, t == 0);
        // S^T of the next tile may overwrite P^T now
        if (t + 1 < n_q) {
          ok = mbar_wait_warp(bar(L::kQFull + st_n), ph_n, abort_flag, kSiteBase + 7);
          if (ragged_q(t + 1)) ok = ok && mbar_wait_warp(bar(L::kQdoFix), 0, abort_flag, kSiteBase + 22);
          if (!ok) break;
          issue_kmajor(kColS, k_km, q_km0 + st_n * kStageStep);
          mma_commit(leader, bar(L::kSFull));
        }
        // dK += dS^T Q
        ok = mbar_wait_warp(bar(L::kDsReady), t & 1, abort_flag, kSiteBase + 8);
        if (!ok) break;
        tc_fence_after_sync();
        issue_acc(kColDk, kColDp, q_mn, t == 0);
        // dQ_i = dS K (needs the previous dQ tile drained out of TMEM)
        ok = mbar_wait_warp(bar(L::kDqEmpty), (t & 1) ^ 1, abort_flag, kSiteBase + 9);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < kBwdTileKV / 16; ++kk) {
          mma_ss(leader, tmem + kColDq, ds_mn + (uint64_t)(kk * (2048 >> 4)), k_mn + (uint64_t)(kk * (2048 >> 4)), idesc_dq,
                 kk > 0);
        }
        mma_commit(leader, bar(L::kDqFull));
        mma_commit(leader, bar(L::kQEmpty + st));
        mma_commit(leader, bar(L::kDoEmpty + st));
        if (t + 1 < n_q) {
          if (kDqAliased) {
            // dQ_i sits in the dP^T columns: wait until it has been drained
            ok = mbar_wait_warp(bar(L::kDqEmpty), t & 1, abort_flag, kSiteBase + 10);
            if (!ok) break;
            tc_fence_after_sync();
          }
          ok = mbar_wait_warp(bar(L::kDoFull + st_n), ph_n, abort_flag, kSiteBase + 11);
          if (!ok) break;
          issue_kmajor(kColDp, v_km, do_km0 + st_n * kStageStep);
          mma_commit(leader, bar(L::kDpFull));
        }
      }
      if (ok) mma_commit(leader, bar(L::kDkvFull));
    }
  } else if (warp < 8) {
    // ============================================================ compute groups
    const int g = warp >> 2;                              // which half of the query columns
    const int lane_row = (warp & 3) * 32 + lane;          // key row within the tile == TMEM lane
    const int kv = kv0 + lane_row;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem + lane_addr + kColS + 64 * g;
    const uint32_t dp_addr = tmem + lane_addr + kColDp + 64 * g;
    const float c1 = p.scale * kLog2e;
    float c0 = p.bias ? p.bias[b] : p.bias_scalar;
    if (p.score_mod && kv < p.Tk) c0 += p.score_mod[(int64_t)b * p.Tk + kv];
    c0 *= kLog2e;
    const bool row_ok = kv < Lk;
    const uint32_t ds_row = smem_base + L::kDsOff + g * 16384 + lane_row * 128;
    const uint32_t sw = (uint32_t)(lane_row & 7);
    bool ok = true;

    for (int t = 0; t < n_q; ++t) {
      const int qc0 = (i_begin + t) * kBwdTileQ + 64 * g;  // first query index of my columns
      // valid(q) for this key row: q_lo <= q < Lq
      const int q_lo = p.causal ? kv : 0;
      const bool need_mask = !row_ok || (qc0 + 64 > Lq) || (p.causal && qc0 < kv0 + kBwdTileKV - 1);
      float pv[64];
      ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kSFull), t & 1, abort_flag, kSiteBase + 12));
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t rbuf[2][32];
      tmem_ld32(s_addr, rbuf[0]);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t(&r)[32] = rbuf[c];
        tmem_ld_wait_for(r);
        if (c == 0) tmem_ld32(s_addr + 32, rbuf[1]);
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 t = __ffma2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])),
                                      make_float2(c1, c1), make_float2(c0, c0));
          float2 pe = sigmoid2_from_log2<kBF16>(t);
          if (need_mask) {
            const int q = qc0 + c * 32 + 2 * i;
            pe.x = (row_ok && q >= q_lo && q < Lq) ? pe.x : 0.0f;
            pe.y = (row_ok && q + 1 >= q_lo && q + 1 < Lq) ? pe.y : 0.0f;
          }
          pv[c * 32 + 2 * i] = pe.x;
          pv[c * 32 + 2 * i + 1] = pe.y;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = pack2<kBF16>(pv[c * 32 + 2 * i], pv[c * 32 + 2 * i + 1]);
        tmem_st16(s_addr + c * 16, pk);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(bar(L::kPReady));

      ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kDpFull), t & 1, abort_flag, kSiteBase + 13));
      if (!ok) break;
      if (t > 0) {
        // the shared-memory copy of dS is still being read by the previous dQ MMA until then
        ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kDqFull), (t - 1) & 1, abort_flag, kSiteBase + 14));
        if (!ok) break;
      }
      tc_fence_after_sync();
      tmem_ld32(dp_addr, rbuf[0]);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t(&r)[32] = rbuf[c];
        tmem_ld_wait_for(r);
        if (c == 0) tmem_ld32(dp_addr + 32, rbuf[1]);
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 pp = make_float2(pv[c * 32 + 2 * i], pv[c * 32 + 2 * i + 1]);
          // dS = P (1 - P) dP = (P - P^2) dP
          const float2 w = __ffma2_rn(make_float2(-pp.x, -pp.y), pp, pp);
          float2 d = __fmul2_rn(w, make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])));
          if (need_mask) {
            d.x = (pp.x != 0.0f) ? d.x : 0.0f;  // masked elements have P exactly 0; keeps NaN/Inf padding out
            d.y = (pp.y != 0.0f) ? d.y : 0.0f;
          }
          pk[i] = pack2<kBF16>(d.x, d.y);
        }
        tmem_st16(dp_addr + c * 16, pk);
        // shared-memory copy for the dQ GEMM: row = key, 64 query columns per 128-byte swizzled line
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const uint32_t chunk = (uint32_t)(4 * c + m) ^ sw;
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(ds_row + chunk * 16), "r"(pk[4 * m]),
                       "r"(pk[4 * m + 1]), "r"(pk[4 * m + 2]), "r"(pk[4 * m + 3])
                       : "memory");
        }
      }
      fence_proxy_async_smem();
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(bar(L::kDsReady));
    }

    // ------------------------------------------------------------ epilogue: group 0 -> dV, group 1 -> dK
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kDkvFull), 0, abort_flag, kSiteBase + 15));
    if (ok) {
      tc_fence_after_sync();
      const uint32_t acc_addr = tmem + lane_addr + (g == 0 ? kColDv : kColDk);
      const float mul = (g == 0) ? 1.0f : p.scale;
      uint8_t* out_row = (g == 0 ? dv_base + 2 * (int64_t)kv * p.dv_st : dk_base + 2 * (int64_t)kv * p.dk_st);
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32_sync(acc_addr + c * 32, r);
        if (kv < p.Tk) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 w;
            w.x = pack2<kBF16>(mul * __uint_as_float(r[8 * q4 + 0]), mul * __uint_as_float(r[8 * q4 + 1]));
            w.y = pack2<kBF16>(mul * __uint_as_float(r[8 * q4 + 2]), mul * __uint_as_float(r[8 * q4 + 3]));
            w.z = pack2<kBF16>(mul * __uint_as_float(r[8 * q4 + 4]), mul * __uint_as_float(r[8 * q4 + 5]));
            w.w = pack2<kBF16>(mul * __uint_as_float(r[8 * q4 + 6]), mul * __uint_as_float(r[8 * q4 + 7]));
            if (!row_ok) w = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(out_row + 64 * c + 16 * q4) = w;
          }
        }
      }
    }
  } else if (warp < 12) {
    // ============================================================ dQ drain
    const int lane_row = (warp & 3) * 32 + lane;  // query row within the tile
    const uint32_t dq_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + kColDq;
    bool ok = true;
    for (int t = 0; t < n_q; ++t) {
      const int q = (i_begin + t) * kBwdTileQ + lane_row;
      float* dst = p.dq_acc + (((int64_t)b * p.Tq + q) * p.H + h) * D;
      ok = __all_sync(0xffffffffu, mbar_wait(bar(L::kDqFull), t & 1, abort_flag, kSiteBase + 16));
      if (!ok) break;
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32_sync(dq_addr + c * 32, r);
        if (c == D / 32 - 1) {
          // everything is in registers: hand the TMEM columns back before the slow part
          tc_fence_before_sync();
          mbar_arrive(bar(L::kDqEmpty));
        }
        if (q < Lq) {
#pragma unroll
          for (int v4 = 0; v4 < 8; ++v4) {
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + c * 32 + v4 * 4),
                         "f"(__uint_as_float(r[4 * v4])), "f"(__uint_as_float(r[4 * v4 + 1])),
                         "f"(__uint_as_float(r[4 * v4 + 2])), "f"(__uint_as_float(r[4 * v4 + 3]))
                         : "memory");
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 13) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
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
