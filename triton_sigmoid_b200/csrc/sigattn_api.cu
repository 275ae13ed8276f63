// Host side of the C ABI declared in include/sigattn_b200.h: argument checks, TMA tensor
// maps, kernel selection and launches.  No device memory is allocated here.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <algorithm>
#include <atomic>
#include <mutex>
#include <stdio.h>
#include <string.h>

#include "../../include/sigattn_b200.h"
#include "bwd_kernel.cuh"
#include "bwd_stream_kernel.cuh"
#include "f32_kernels.cuh"
#include "fwd_kernel.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define SIG_CUDA(expr)                                                                            \
  do {                                                                                            \
    cudaError_t e_ = (expr);                                                                      \
    if (e_ != cudaSuccess) return fail(-100, "%s failed: %s", #expr, cudaGetErrorString(e_));     \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Tensor map over a (B, T, H, D) tensor with element strides {sb, st, sh} and unit stride in
// D.  TMA dimensions are ordered (d, h, t, b); one box is 64 elements of d by `box_rows`
// tokens of one head of one batch, written to shared memory with the 128-byte swizzle.
// Rows at or beyond T read as zeros.
int make_map(CUtensorMap* m, const void* base, int dtype, int B, int T, int H, int D, const int64_t* strides,
             int box_rows, const char* name) {
  // Encoding a tensor map is a driver call of a microsecond or two, and a training loop calls with the same
  // tensors (or the same allocator blocks) again and again: a small per-thread cache keyed by everything the
  // encoding depends on.
  struct Key {
    const void* base;
    int dtype, B, T, H, D, box_rows;
    int64_t s0, s1, s2;
    bool operator==(const Key& o) const {
      return base == o.base && dtype == o.dtype && B == o.B && T == o.T && H == o.H && D == o.D && box_rows == o.box_rows &&
             s0 == o.s0 && s1 == o.s1 && s2 == o.s2;
    }
  };
  constexpr int kCacheEntries = 16;
  struct Entry { Key key; CUtensorMap map; bool valid; };
  thread_local Entry cache[kCacheEntries] = {};
  thread_local int next_victim = 0;
  const Key key{base, dtype, B, T, H, D, box_rows, strides[0], strides[1], strides[2]};
  for (int i = 0; i < kCacheEntries; ++i)
    if (cache[i].valid && cache[i].key == key) {
      *m = cache[i].map;
      return 0;
    }
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return fail(-101, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return fail(-3, "%s: base pointer must be 16-byte aligned", name);
  for (int i = 0; i < 3; ++i)
    if (strides[i] <= 0 || (strides[i] * 2) % 16 != 0)
      return fail(-3, "%s: stride %d (%lld elements) must be positive and a multiple of 8 elements", name, i,
                  (long long)strides[i]);
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)T, (cuuint64_t)B};
  cuuint64_t gstr[3] = {(cuuint64_t)strides[2] * 2, (cuuint64_t)strides[1] * 2, (cuuint64_t)strides[0] * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(m, dtype == SIGATTN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   const_cast<void*>(base), dims, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-102, "%s: cuTensorMapEncodeTiled failed with CUresult %d", name, (int)r);
  Entry& e = cache[next_victim];
  next_victim = (next_victim + 1) % kCacheEntries;
  e.key = key;
  e.map = *m;
  e.valid = true;
  return 0;
}

int check_common(const SigAttnParams* p, bool backward) {
  if (!p) return fail(-1, "params is NULL");
  if (p->struct_bytes != sizeof(SigAttnParams))
    return fail(-1, "struct_bytes %u != sizeof(SigAttnParams) %zu (ABI mismatch)", p->struct_bytes,
                sizeof(SigAttnParams));
  if (p->dtype != SIGATTN_FP16 && p->dtype != SIGATTN_BF16 && p->dtype != SIGATTN_FP32)
    return fail(-2, "unsupported dtype %d (fp16=0, bf16=1, fp32=2)", p->dtype);
  if (p->D != 64 && p->D != 128) return fail(-2, "unsupported head dimension %d (64 or 128)", p->D);
  if (p->B < 0 || p->H < 0 || p->Tq < 0 || p->Tk < 0) return fail(-2, "negative extent");
  if (p->H > 65535 || p->B > 65535) return fail(-2, "B and H must not exceed 65535");
  const bool packed = p->cu_seqlens_q || p->cu_seqlens_k;
  if (packed) {
    if (!p->cu_seqlens_q || !p->cu_seqlens_k) return fail(-1, "packed layout needs both cu_seqlens_q and cu_seqlens_k");
    if (p->seq_lens_q || p->seq_lens_k) return fail(-2, "packed layout: seq_lens_q / seq_lens_k must be NULL");
    if (p->total_q < 0 || p->total_k < 0) return fail(-2, "negative total_q / total_k");
  }
  if (p->B == 0 || p->H == 0) return 1;  // nothing to do
  if (!p->q || !p->k || !p->v) return fail(-1, "q, k, v must not be NULL");
  if (!backward && !p->o) return fail(-1, "o must not be NULL");
  if (backward && (!p->dout || !p->dq || !p->dk || !p->dv)) return fail(-1, "dout, dq, dk, dv must not be NULL");
  return 0;
}

bool is_contiguous(const int64_t* s, int T, int H, int D) {
  return s[2] == D && s[1] == (int64_t)H * D && s[0] == (int64_t)T * H * D;
}

// Extents of the tensors as the tensor maps, the accumulator and the fills see them: packed tensors are
// one "batch" of total_q / total_k rows.
struct Extents {
  int B, Tq, Tk;
  bool packed;
};
Extents extents(const SigAttnParams* p) {
  const bool packed = p->cu_seqlens_q != nullptr;
  return Extents{packed ? 1 : p->B, packed ? p->total_q : p->Tq, packed ? p->total_k : p->Tk, packed};
}
// {batch, token, head} strides with a usable batch stride when the tensor is packed
struct Strides3 {
  int64_t s[3];
};
Strides3 map_strides(const int64_t* strides, int T, bool packed) {
  Strides3 r{{strides[0], strides[1], strides[2]}};
  if (packed) r.s[0] = (int64_t)(T > 0 ? T : 1) * strides[1];
  return r;
}

// Zero-fill a (B,T,H,D) tensor; only used for degenerate problems (no keys / no queries).
int zero_fill(void* ptr, const int64_t* strides, int B, int T, int H, int D, int dtype, cudaStream_t stream,
              const char* name) {
  if (T == 0) return 0;
  if (!is_contiguous(strides, T, H, D)) return fail(-2, "%s: an empty problem needs a contiguous output", name);
  SIG_CUDA(cudaMemsetAsync(ptr, 0, (size_t)B * T * H * D * (dtype == SIGATTN_FP32 ? 4 : 2), stream));
  return 0;
}

struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  cudaError_t enter(int dev) {
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return e;
    // Always set the device: on a host thread that has made no runtime call yet (an autograd
    // worker, say) this is what binds the primary context, which the driver-level tensor-map
    // encoder needs.
    e = cudaSetDevice(dev);
    switched = (e == cudaSuccess) && prev != dev;
    return e;
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

// Opt-in to the kernel's dynamic shared memory: once per kernel and device (`K` is a distinct type per
// kernel signature only, so the flags are keyed by the kernel's address).
template <typename K>
int set_smem(K kernel, int bytes, int device) {
  constexpr int kMaxKernels = 64, kMaxDevices = 64;
  static std::mutex mu;
  static const void* seen[kMaxKernels] = {};
  static bool done[kMaxKernels][kMaxDevices] = {};
  if (device >= 0 && device < kMaxDevices) {
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < kMaxKernels; ++i) {
      if (seen[i] == nullptr) seen[i] = reinterpret_cast<const void*>(kernel);
      if (seen[i] == reinterpret_cast<const void*>(kernel)) {
        if (done[i][device]) return 0;
        SIG_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
        done[i][device] = true;
        return 0;
      }
    }
  }
  SIG_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  return 0;
}

// Work-item counters of the persistent kernels (forward and backward): a ring of (next item, finished CTAs) pairs.
// Each launch takes the next pair; the kernel leaves its pair at zero when its last CTA finishes,
// so a pair is only in doubt if more launches than the pool holds are in flight at once on one device.
// Launches recorded into a stream capture keep their pair for every replay of the graph, so they draw
// from a pool of their own that eager launches never touch.
constexpr int kTicketSlots = 1024;
constexpr int kEagerTicketSlots = 768;  // the remaining 256 serve launches made under stream capture
__device__ unsigned int g_item_tickets[2 * kTicketSlots];

// Host-visible copies of the devices' health words (see g_status_mirror in ptx.cuh): one page of this
// library's own host data, pinned and mapped once per process.  A kernel writes its device's entry
// only when it abandons a wait; every attention call reads it (a plain host load) before launching.
constexpr int kMaxMirrorDevices = 64;
alignas(4096) volatile int g_host_status[1024];
bool g_host_status_mapped = false;

struct FwdDeviceInfo {
  unsigned int* tickets = nullptr;
  int n_sm = 0;
};

// Device address of the counters and the SM count, looked up once per device (which must be current).
int fwd_device_info(int device, FwdDeviceInfo* out) {
  constexpr int kMaxDevices = 64;
  static FwdDeviceInfo cached[kMaxDevices];
  static std::mutex mu;
  if (device < 0 || device >= kMaxDevices) return fail(-2, "device ordinal %d out of range", device);
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[device].tickets) {
    unsigned int* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_item_tickets);
    if (e != cudaSuccess || !ptr)
      return fail(-100, "cudaGetSymbolAddress(work-item counters) failed on device %d: %s", device,
                  cudaGetErrorString(e));
    int n_sm = 0;
    SIG_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, device));
    if (n_sm <= 0) return fail(-100, "device %d reports %d multiprocessors", device, n_sm);
    // health-word mirror: best effort (without it failures are still reported by sigattn_device_status)
    if (!g_host_status_mapped) {
      if (cudaHostRegister(const_cast<int*>(g_host_status), sizeof(g_host_status),
                           cudaHostRegisterPortable | cudaHostRegisterMapped) == cudaSuccess)
        g_host_status_mapped = true;
      else
        (void)cudaGetLastError();
    }
    if (g_host_status_mapped && device < kMaxMirrorDevices) {
      int* dev_view = nullptr;
      if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&dev_view), const_cast<int*>(&g_host_status[device]), 0) ==
              cudaSuccess && dev_view) {
        volatile int* as_volatile = dev_view;
        if (cudaMemcpyToSymbol(sigattn::g_status_mirror, &as_volatile, sizeof(as_volatile)) != cudaSuccess)
          (void)cudaGetLastError();
      } else {
        (void)cudaGetLastError();
      }
    }
    cached[device].n_sm = n_sm;
    cached[device].tickets = ptr;
  }
  *out = cached[device];
  return 0;
}

// Non-zero when a kernel of this library has abandoned a wait on `device` and nobody has read the
// failure yet (sigattn_device_status reads and clears it).
int pending_failure(int device) {
  if (device < 0 || device >= kMaxMirrorDevices) return 0;
  return g_host_status[device];
}
#define SIG_REFUSE_IF_SICK(p)                                                                               \
  do {                                                                                                      \
    if (int site_ = pending_failure((p)->device))                                                           \
      return fail(-5, "device %d: a kernel gave up on a bounded wait (site 0x%x); results since then are "  \
                      "undefined and launches are refused until sigattn_device_status() has been called",   \
                  (p)->device, site_);                                                                      \
  } while (0)

// (batch, head) pairs per scheduling group of the persistent kernels.  Under a causal mask the items of
// one head differ in weight, and handing out the heavy items of many heads first balances the CTAs; the
// group is limited so that what its heads stream per item (`bytes_per_head`) stays within the L2.
// Without a causal mask the plain order is kept.
int schedule_group(bool causal, int64_t n_bh, int64_t bytes_per_head, int64_t l2_budget) {
  if (!causal || n_bh <= 1) return 1;
  int64_t g = l2_budget / (bytes_per_head > 0 ? bytes_per_head : 1);
  if (g < 1) g = 1;
  if (g > n_bh) g = n_bh;
  return (int)g;
}

// The pair of counters for one launch on `stream`.
unsigned int* next_ticket_pair(const FwdDeviceInfo& info, int device, cudaStream_t stream) {
  static std::atomic<unsigned int> next_eager[64], next_captured[64];
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) {
    (void)cudaGetLastError();
    st = cudaStreamCaptureStatusNone;
  }
  if (st == cudaStreamCaptureStatusNone) return info.tickets + 2 * (next_eager[device].fetch_add(1u) % kEagerTicketSlots);
  return info.tickets + 2 * (kEagerTicketSlots + next_captured[device].fetch_add(1u) % (kTicketSlots - kEagerTicketSlots));
}

template <int D, bool kBF16, bool kScoreMod, bool kAccurate>
int launch_fwd(const SigAttnParams* p, const CUtensorMap& qm, const CUtensorMap& km, const CUtensorMap& vm) {
  using namespace sigattn;
  auto kernel = sigattn_fwd_kernel<D, kBF16, kScoreMod, kAccurate>;
  constexpr int smem = FwdSmem<D>::kDynBytes;
  if (int rc = set_smem(kernel, smem, p->device)) return rc;
  FwdParams fp;
  fp.o = p->o;
  fp.o_sb = p->o_strides[0];
  fp.o_st = p->o_strides[1];
  fp.o_sh = p->o_strides[2];
  fp.lens_q = p->seq_lens_q;
  fp.lens_k = p->seq_lens_k;
  fp.cu_q = p->cu_seqlens_q;
  fp.cu_k = p->cu_seqlens_k;
  fp.bias = p->bias;
  fp.score_mod = p->score_mod;
  fp.scale = p->scale;
  fp.bias_scalar = p->bias_scalar;
  if (p->flags & SIGATTN_BIAS_NEG_LOG_LK) { fp.bias = nullptr; fp.bias_scalar = nanf(""); }  // see item_bias()
  fp.B = p->B;
  fp.H = p->H;
  fp.Tq = p->Tq;
  fp.Tk = p->Tk;
  fp.causal = (p->flags & SIGATTN_CAUSAL) ? 1 : 0;
  fp.n_qblk = (p->Tq + kFwdBlockM - 1) / kFwdBlockM;
  const int64_t n_items = (int64_t)fp.n_qblk * p->H * p->B;
  if (n_items > INT32_MAX) return fail(-2, "too many (batch, head, query block) items: %lld", (long long)n_items);
  fp.n_items = (int)n_items;
  // K and V of one head, half of the L2 for them
  fp.group = schedule_group(fp.causal != 0, (int64_t)p->B * p->H, (int64_t)p->Tk * D * 2 * 2, 64ll << 20);
  FwdDeviceInfo info;
  if (int rc = fwd_device_info(p->device, &info)) return rc;
  fp.ticket = next_ticket_pair(info, p->device, static_cast<cudaStream_t>(p->stream));
  // persistent: one CTA per SM (the kernel's shared memory allows no more), fewer when there are fewer items
  dim3 grid((unsigned int)std::min<int64_t>(n_items, info.n_sm));
  cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  if (p->ev_main_start) SIG_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(p->ev_main_start), stream));
  kernel<<<grid, kFwdThreads, smem, stream>>>(qm, km, vm, fp);
  SIG_CUDA(cudaGetLastError());
  if (p->ev_main_stop) SIG_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(p->ev_main_stop), stream));
  return 0;
}

// The default backward: the fused 5-GEMM kernel with fp32 dQ reductions into a workspace (bwd_kernel.cuh).
template <int D, bool kBF16, bool kAccurate>
int launch_bwd_fused(const SigAttnParams* p, const CUtensorMap& qm, const CUtensorMap& km, const CUtensorMap& vm,
                     const CUtensorMap& dom) {
  using namespace sigattn;
  cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  const Extents ex = extents(p);
  const size_t need = sigattn_bwd_workspace_bytes(ex.B, ex.Tq, p->H, p->D);
  if (p->workspace_bytes < need || (need && !p->workspace))
    return fail(-4, "backward workspace too small: %zu bytes given, %zu needed", p->workspace_bytes, need);
  if ((reinterpret_cast<uintptr_t>(p->workspace) & 15u) != 0) return fail(-3, "workspace must be 16-byte aligned");
  float* dq_acc = static_cast<float*>(p->workspace);
  SIG_CUDA(cudaMemsetAsync(dq_acc, 0, need, stream));

  BwdParams bp;
  bp.dq_acc = dq_acc;
  bp.dk = p->dk;
  bp.dv = p->dv;
  bp.dk_sb = p->dk_strides[0]; bp.dk_st = p->dk_strides[1]; bp.dk_sh = p->dk_strides[2];
  bp.dv_sb = p->dv_strides[0]; bp.dv_st = p->dv_strides[1]; bp.dv_sh = p->dv_strides[2];
  bp.lens_q = p->seq_lens_q;
  bp.lens_k = p->seq_lens_k;
  bp.cu_q = p->cu_seqlens_q;
  bp.cu_k = p->cu_seqlens_k;
  bp.bias = p->bias;
  bp.score_mod = p->score_mod;
  bp.scale = p->scale;
  bp.bias_scalar = p->bias_scalar;
  if (p->flags & SIGATTN_BIAS_NEG_LOG_LK) { bp.bias = nullptr; bp.bias_scalar = nanf(""); }  // see item_bias()
  bp.B = p->B; bp.H = p->H; bp.Tq = p->Tq; bp.Tk = p->Tk;
  bp.causal = (p->flags & SIGATTN_CAUSAL) ? 1 : 0;
  bp.n_kvblk = (p->Tk + kBwdTileKV - 1) / kBwdTileKV;
  const int64_t n_items = (int64_t)bp.n_kvblk * p->H * p->B;
  if (n_items > INT32_MAX) return fail(-2, "too many (batch, head, key tile) items: %lld", (long long)n_items);
  bp.n_items = (int)n_items;
  // Q, dO and the fp32 dQ accumulator of one head; a quarter of the L2 (measured: larger groups cost the
  // reductions their locality, a few heads already balance the CTAs)
  bp.group = schedule_group(bp.causal != 0, (int64_t)p->B * p->H, (int64_t)p->Tq * D * (2 + 2 + 4), 32ll << 20);
  FwdDeviceInfo info;
  if (int rc = fwd_device_info(p->device, &info)) return rc;
  bp.ticket = next_ticket_pair(info, p->device, stream);

  {
    auto kernel = sigattn_bwd_kernel<D, kBF16, kAccurate>;
    constexpr int smem = BwdSmem<D>::kDynBytes;
    if (int rc = set_smem(kernel, smem, p->device)) return rc;
    // persistent: one CTA per SM (the kernel's shared memory allows no more), fewer when there are fewer items
    dim3 grid((unsigned int)std::min<int64_t>(n_items, info.n_sm));
    if (p->ev_main_start) SIG_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(p->ev_main_start), stream));
    kernel<<<grid, kBwdThreads<D>, smem, stream>>>(qm, km, vm, dom, bp);
    SIG_CUDA(cudaGetLastError());
    if (p->ev_main_stop) SIG_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(p->ev_main_stop), stream));
  }
  {
    // dQ = scale * accumulator, rounded to the 16-bit type
    DqConvertParams cp;
    cp.acc = dq_acc;
    cp.dq = p->dq;
    cp.sb = p->dq_strides[0]; cp.st = p->dq_strides[1]; cp.sh = p->dq_strides[2];
    cp.B = ex.B; cp.T = ex.Tq; cp.H = p->H;
    cp.scale = p->scale;
    const long long chunks = (long long)ex.B * ex.Tq * p->H * (D / 8);
    const int threads = 256;
    const long long blocks_ll = (chunks + threads - 1) / threads;
    const int blocks = (int)(blocks_ll > 148LL * 64 ? 148LL * 64 : blocks_ll);
    sigattn_dq_convert_kernel<D, kBF16><<<blocks, threads, 0, stream>>>(cp);
    SIG_CUDA(cudaGetLastError());
  }
  return 0;
}

// The split backward (SIGATTN_BWD_SPLIT): the streaming kernel of bwd_stream_kernel.cuh, once in dK/dV mode
// and once in dQ mode.  No workspace, no atomics, deterministic.
template <int D, bool kBF16, bool kDKV, bool kAccurate>
int launch_bwd_stream_mode(const SigAttnParams* p, const CUtensorMap& r1, const CUtensorMap& r2, const CUtensorMap& c1,
                           const CUtensorMap& c2, const FwdDeviceInfo& info) {
  using namespace sigattn;
  cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  BwdStreamParams bp;
  if (kDKV) {
    bp.out1 = p->dk; bp.o1_sb = p->dk_strides[0]; bp.o1_st = p->dk_strides[1]; bp.o1_sh = p->dk_strides[2];
    bp.out2 = p->dv; bp.o2_sb = p->dv_strides[0]; bp.o2_st = p->dv_strides[1]; bp.o2_sh = p->dv_strides[2];
    bp.lens_r = p->seq_lens_k; bp.lens_c = p->seq_lens_q;
    bp.cu_r = p->cu_seqlens_k; bp.cu_c = p->cu_seqlens_q;
    bp.Tr = p->Tk; bp.Tc = p->Tq;
  } else {
    bp.out1 = p->dq; bp.o1_sb = p->dq_strides[0]; bp.o1_st = p->dq_strides[1]; bp.o1_sh = p->dq_strides[2];
    bp.out2 = nullptr; bp.o2_sb = bp.o2_st = bp.o2_sh = 0;
    bp.lens_r = p->seq_lens_q; bp.lens_c = p->seq_lens_k;
    bp.cu_r = p->cu_seqlens_q; bp.cu_c = p->cu_seqlens_k;
    bp.Tr = p->Tq; bp.Tc = p->Tk;
  }
  bp.bias = p->bias;
  bp.score_mod = p->score_mod;
  bp.scale = p->scale;
  bp.bias_scalar = p->bias_scalar;
  if (p->flags & SIGATTN_BIAS_NEG_LOG_LK) { bp.bias = nullptr; bp.bias_scalar = nanf(""); }  // see item_bias()
  bp.B = p->B; bp.H = p->H; bp.Tk = p->Tk;
  bp.causal = (p->flags & SIGATTN_CAUSAL) ? 1 : 0;
  bp.n_rblk = (bp.Tr + kBsTile - 1) / kBsTile;
  const int64_t n_items = (int64_t)bp.n_rblk * p->H * p->B;
  if (n_items > INT32_MAX) return fail(-2, "too many (batch, head, tile) items: %lld", (long long)n_items);
  bp.n_items = (int)n_items;
  // what one head streams per item (the two streamed tensors), half of the L2 for a group
  bp.group = schedule_group(bp.causal != 0, (int64_t)p->B * p->H, (int64_t)bp.Tc * D * 2 * 2, 64ll << 20);
  bp.ticket = next_ticket_pair(info, p->device, stream);
  auto kernel = sigattn_bwd_stream_kernel<D, kBF16, kDKV, kAccurate>;
  constexpr int smem = BsSmem<D, kDKV>::kDynBytes;
  if (int rc = set_smem(kernel, smem, p->device)) return rc;
  dim3 grid((unsigned int)std::min<int64_t>(n_items, info.n_sm));
  kernel<<<grid, kBsThreads, smem, stream>>>(r1, r2, c1, c2, bp);
  SIG_CUDA(cudaGetLastError());
  return 0;
}

template <int D, bool kBF16, bool kAccurate>
int launch_bwd_stream(const SigAttnParams* p, const CUtensorMap& qm, const CUtensorMap& km, const CUtensorMap& vm,
                      const CUtensorMap& dom) {
  FwdDeviceInfo info;
  if (int rc = fwd_device_info(p->device, &info)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  if (p->ev_main_start) SIG_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(p->ev_main_start), stream));
  if (int rc = launch_bwd_stream_mode<D, kBF16, true, kAccurate>(p, km, vm, qm, dom, info)) return rc;
  if (int rc = launch_bwd_stream_mode<D, kBF16, false, kAccurate>(p, qm, dom, km, vm, info)) return rc;
  if (p->ev_main_stop) SIG_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(p->ev_main_stop), stream));
  return 0;
}

// Scratch of sigattn_bwd_static_scratch: lives in the device image of this library.
static __device__ __align__(256) float g_static_dq_scratch[SIGATTN_STATIC_SCRATCH_ELEMS];

// In host code the name above is only a handle for the runtime, not a device address; the
// address valid on `device` is looked up once per device (with that device current) and cached.
int static_scratch_ptr(int device, float** out) {
  constexpr int kMaxDevices = 64;
  static float* cached[kMaxDevices] = {};
  static std::mutex mu;
  if (device < 0 || device >= kMaxDevices) return fail(-2, "device ordinal %d out of range", device);
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[device]) {
    int cur = -1;
    SIG_CUDA(cudaGetDevice(&cur));
    if (cur != device) return fail(-100, "internal: device %d is not current (current is %d)", device, cur);
    float* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_dq_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(-100, "cudaGetSymbolAddress(static dQ scratch) failed on device %d: %s", device, cudaGetErrorString(e));
    cached[device] = ptr;
  }
  *out = cached[device];
  return 0;
}

// float32 tensors: the exact FMA-pipe kernels (no tensor maps, no workspace).
template <int D>
int launch_f32_d(const SigAttnParams* p, bool backward) {
  using namespace sigattn;
  F32Params fp = {};
  fp.q = static_cast<const float*>(p->q);
  fp.k = static_cast<const float*>(p->k);
  fp.v = static_cast<const float*>(p->v);
  fp.dout = static_cast<const float*>(p->dout);
  fp.o = static_cast<float*>(p->o);
  fp.dq = static_cast<float*>(p->dq);
  fp.dk = static_cast<float*>(p->dk);
  fp.dv = static_cast<float*>(p->dv);
  fp.q_sb = p->q_strides[0]; fp.q_st = p->q_strides[1]; fp.q_sh = p->q_strides[2];
  fp.k_sb = p->k_strides[0]; fp.k_st = p->k_strides[1]; fp.k_sh = p->k_strides[2];
  fp.v_sb = p->v_strides[0]; fp.v_st = p->v_strides[1]; fp.v_sh = p->v_strides[2];
  fp.o_sb = p->o_strides[0]; fp.o_st = p->o_strides[1]; fp.o_sh = p->o_strides[2];
  fp.do_sb = p->do_strides[0]; fp.do_st = p->do_strides[1]; fp.do_sh = p->do_strides[2];
  fp.dq_sb = p->dq_strides[0]; fp.dq_st = p->dq_strides[1]; fp.dq_sh = p->dq_strides[2];
  fp.dk_sb = p->dk_strides[0]; fp.dk_st = p->dk_strides[1]; fp.dk_sh = p->dk_strides[2];
  fp.dv_sb = p->dv_strides[0]; fp.dv_st = p->dv_strides[1]; fp.dv_sh = p->dv_strides[2];
  fp.lens_q = p->seq_lens_q;
  fp.lens_k = p->seq_lens_k;
  fp.cu_q = p->cu_seqlens_q;
  fp.cu_k = p->cu_seqlens_k;
  fp.bias = p->bias;
  fp.score_mod = p->score_mod;
  fp.scale = p->scale;
  fp.bias_scalar = p->bias_scalar;
  if (p->flags & SIGATTN_BIAS_NEG_LOG_LK) { fp.bias = nullptr; fp.bias_scalar = nanf(""); }  // see item_bias()
  fp.B = p->B; fp.H = p->H; fp.Tq = p->Tq; fp.Tk = p->Tk;
  fp.causal = (p->flags & SIGATTN_CAUSAL) ? 1 : 0;
  cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
  const unsigned int n_q = (unsigned int)((p->Tq + kF32Tile - 1) / kF32Tile);
  const unsigned int n_k = (unsigned int)((p->Tk + kF32Tile - 1) / kF32Tile);
  if (p->ev_main_start) SIG_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(p->ev_main_start), stream));
  if (!backward) {
    auto kernel = sigattn_fwd_f32_kernel<D>;
    if (int rc = set_smem(kernel, F32Smem<D>::kFwdBytes, p->device)) return rc;
    kernel<<<dim3(n_q, p->H, p->B), kF32Threads, F32Smem<D>::kFwdBytes, stream>>>(fp);
    SIG_CUDA(cudaGetLastError());
  } else {
    auto kdkdv = sigattn_bwd_dkdv_f32_kernel<D>;
    auto kdq = sigattn_bwd_dq_f32_kernel<D>;
    if (int rc = set_smem(kdkdv, F32Smem<D>::kDkdvBytes, p->device)) return rc;
    if (int rc = set_smem(kdq, F32Smem<D>::kDqBytes, p->device)) return rc;
    kdkdv<<<dim3(n_k, p->H, p->B), kF32Threads, F32Smem<D>::kDkdvBytes, stream>>>(fp);
    SIG_CUDA(cudaGetLastError());
    kdq<<<dim3(n_q, p->H, p->B), kF32Threads, F32Smem<D>::kDqBytes, stream>>>(fp);
    SIG_CUDA(cudaGetLastError());
  }
  if (p->ev_main_stop) SIG_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(p->ev_main_stop), stream));
  return 0;
}

int launch_f32(const SigAttnParams* p, bool backward) {
  struct Tensor { const void* ptr; const int64_t* strides; const char* name; };
  const Tensor fwd_t[] = {{p->q, p->q_strides, "q"}, {p->k, p->k_strides, "k"}, {p->v, p->v_strides, "v"}, {p->o, p->o_strides, "o"}};
  const Tensor bwd_t[] = {{p->q, p->q_strides, "q"}, {p->k, p->k_strides, "k"}, {p->v, p->v_strides, "v"},
                          {p->dout, p->do_strides, "dout"}, {p->dq, p->dq_strides, "dq"}, {p->dk, p->dk_strides, "dk"},
                          {p->dv, p->dv_strides, "dv"}};
  const Tensor* ts = backward ? bwd_t : fwd_t;
  const int n = backward ? 7 : 4;
  for (int t = 0; t < n; ++t) {
    if ((reinterpret_cast<uintptr_t>(ts[t].ptr) & 15u) != 0) return fail(-3, "%s: base pointer must be 16-byte aligned", ts[t].name);
    for (int i = 0; i < 3; ++i)
      if (ts[t].strides[i] % 4 != 0) return fail(-3, "%s: strides must be multiples of 4 elements (16 bytes)", ts[t].name);
  }
  return p->D == 64 ? launch_f32_d<64>(p, backward) : launch_f32_d<128>(p, backward);
}

// Self-test of the bounded waits: one warp waits on a barrier that nothing ever arrives on, with a
// limit of a few milliseconds, exactly as a kernel of the library would on a lost signal: the wait
// gives up, records its site in the health word, and the kernel returns normally.
constexpr int kSelfTestSite = 0x30001;
__global__ void sigattn_selftest_wait_kernel(unsigned long long limit_ns, int* gave_up) {
  __shared__ __align__(8) unsigned long long bar_storage;
  __shared__ int abort_flag;
  const uint32_t bar = sigattn::smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    sigattn::mbar_init(bar, 1);
    sigattn::fence_mbar_init();
  }
  __syncthreads();
  const bool ok = sigattn::mbar_wait(bar, 0, &abort_flag, kSelfTestSite, limit_ns);
  if (threadIdx.x == 0) *gave_up = ok ? 0 : 1;
}

}  // namespace

extern "C" {

const char* sigattn_last_error(void) { return g_err; }

int sigattn_query(int what) {
  switch (what) {
    case SIGATTN_Q_ABI_VERSION: return SIGATTN_ABI_VERSION;
    case SIGATTN_Q_SM_ARCH: return 100;
    case SIGATTN_Q_MAX_HEAD_DIM: return 128;
    case SIGATTN_Q_PARAMS_SIZE: return (int)sizeof(SigAttnParams);
    default: return -1;
  }
}

size_t sigattn_bwd_workspace_bytes(int32_t B, int32_t Tq, int32_t H, int32_t D) {
  if (B <= 0 || Tq <= 0 || H <= 0 || D <= 0) return 0;
  return (size_t)B * (size_t)Tq * (size_t)H * (size_t)D * sizeof(float);
}

int sigattn_device_status(int device) {
  DeviceGuard g;
  SIG_CUDA(g.enter(device));
  SIG_CUDA(cudaDeviceSynchronize());
  int v = 0;
  SIG_CUDA(cudaMemcpyFromSymbol(&v, sigattn::g_status_word, sizeof(int)));
  if (v != 0) {
    // A kernel that gave up may have left its work-item counters half used: clear them together
    // with the status, so that the library is usable again after the caller has seen the failure.
    int zero = 0;
    SIG_CUDA(cudaMemcpyToSymbol(sigattn::g_status_word, &zero, sizeof(int)));
    void* tickets = nullptr;
    SIG_CUDA(cudaGetSymbolAddress(&tickets, g_item_tickets));
    SIG_CUDA(cudaMemset(tickets, 0, sizeof(unsigned int) * 2 * kTicketSlots));
  }
  if (device >= 0 && device < kMaxMirrorDevices) g_host_status[device] = 0;
  return v;
}


int sigattn_selftest_bounded_wait(int device, int limit_ms) {
  g_err[0] = 0;
  if (limit_ms < 1 || limit_ms > 1000) return fail(-2, "limit_ms must be in [1, 1000], got %d", limit_ms);
  DeviceGuard g;
  SIG_CUDA(g.enter(device));
  {
    FwdDeviceInfo info;  // first use of the device: also installs the host-visible copy of the health word
    if (int rc = fwd_device_info(device, &info)) return rc;
  }
  int* flag = nullptr;
  SIG_CUDA(cudaMalloc(&flag, sizeof(int)));
  cudaError_t e = cudaMemset(flag, 0xff, sizeof(int));
  int gave_up = -1;
  if (e == cudaSuccess) {
    sigattn_selftest_wait_kernel<<<1, 32>>>((unsigned long long)limit_ms * 1000000ull, flag);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaMemcpy(&gave_up, flag, sizeof(int), cudaMemcpyDeviceToHost);
  cudaFree(flag);
  if (e != cudaSuccess) return fail(-100, "self-test: %s", cudaGetErrorString(e));
  return gave_up;
}

int sigattn_fwd(const SigAttnParams* p) {
  g_err[0] = 0;
  int rc = check_common(p, false);
  if (rc < 0) return rc;
  if (rc == 1) return 0;
  SIG_REFUSE_IF_SICK(p);
  DeviceGuard g;
  SIG_CUDA(g.enter(p->device));
  const Extents ex = extents(p);
  if (ex.Tq == 0 || p->Tq == 0) return 0;
  if (ex.Tk == 0 || p->Tk == 0) {  // no keys at all: the output is all zeros
    const Strides3 os = map_strides(p->o_strides, ex.Tq, ex.packed);
    return zero_fill(p->o, os.s, ex.B, ex.Tq, p->H, p->D, p->dtype, static_cast<cudaStream_t>(p->stream), "o");
  }
  if (p->dtype == SIGATTN_FP32) return launch_f32(p, false);
  CUtensorMap qm, km, vm;
  if ((rc = make_map(&qm, p->q, p->dtype, ex.B, ex.Tq, p->H, p->D, map_strides(p->q_strides, ex.Tq, ex.packed).s, 128, "q"))) return rc;
  if ((rc = make_map(&km, p->k, p->dtype, ex.B, ex.Tk, p->H, p->D, map_strides(p->k_strides, ex.Tk, ex.packed).s, 128, "k"))) return rc;
  if ((rc = make_map(&vm, p->v, p->dtype, ex.B, ex.Tk, p->H, p->D, map_strides(p->v_strides, ex.Tk, ex.packed).s, 128, "v"))) return rc;
  if ((reinterpret_cast<uintptr_t>(p->o) & 15u) != 0) return fail(-3, "o: base pointer must be 16-byte aligned");
  for (int i = ex.packed ? 1 : 0; i < 3; ++i)
    if (p->o_strides[i] % 8 != 0) return fail(-3, "o: strides must be multiples of 8 elements");

  const bool bf = p->dtype == SIGATTN_BF16;
  const bool sm = p->score_mod != nullptr;
  const bool acc = (p->flags & SIGATTN_ACCURATE) != 0;
#define SIG_FWD(DD, BF, SM)                                             \
  do {                                                                  \
    if (acc) return launch_fwd<DD, BF, SM, true>(p, qm, km, vm);        \
    return launch_fwd<DD, BF, SM, false>(p, qm, km, vm);                \
  } while (0)
  if (p->D == 64) {
    if (bf) { if (sm) SIG_FWD(64, true, true); else SIG_FWD(64, true, false); }
    else    { if (sm) SIG_FWD(64, false, true); else SIG_FWD(64, false, false); }
  } else {
    if (bf) { if (sm) SIG_FWD(128, true, true); else SIG_FWD(128, true, false); }
    else    { if (sm) SIG_FWD(128, false, true); else SIG_FWD(128, false, false); }
  }
#undef SIG_FWD
  return fail(-2, "unreachable");
}

int sigattn_bwd(const SigAttnParams* p) {
  g_err[0] = 0;
  int rc = check_common(p, true);
  if (rc < 0) return rc;
  if (rc == 1) return 0;
  SIG_REFUSE_IF_SICK(p);
  DeviceGuard g;
  SIG_CUDA(g.enter(p->device));
  const Extents ex = extents(p);
  if (ex.Tq == 0 || ex.Tk == 0 || p->Tq == 0 || p->Tk == 0) {
    // no query or no key: every gradient is zero
    cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
    if ((rc = zero_fill(p->dq, map_strides(p->dq_strides, ex.Tq, ex.packed).s, ex.B, ex.Tq, p->H, p->D, p->dtype, stream, "dq"))) return rc;
    if ((rc = zero_fill(p->dk, map_strides(p->dk_strides, ex.Tk, ex.packed).s, ex.B, ex.Tk, p->H, p->D, p->dtype, stream, "dk"))) return rc;
    return zero_fill(p->dv, map_strides(p->dv_strides, ex.Tk, ex.packed).s, ex.B, ex.Tk, p->H, p->D, p->dtype, stream, "dv");
  }
  if (p->dtype == SIGATTN_FP32) return launch_f32(p, true);
  CUtensorMap qm, km, vm, dom;
  if ((rc = make_map(&qm, p->q, p->dtype, ex.B, ex.Tq, p->H, p->D, map_strides(p->q_strides, ex.Tq, ex.packed).s, 128, "q"))) return rc;
  if ((rc = make_map(&km, p->k, p->dtype, ex.B, ex.Tk, p->H, p->D, map_strides(p->k_strides, ex.Tk, ex.packed).s, 128, "k"))) return rc;
  if ((rc = make_map(&vm, p->v, p->dtype, ex.B, ex.Tk, p->H, p->D, map_strides(p->v_strides, ex.Tk, ex.packed).s, 128, "v"))) return rc;
  if ((rc = make_map(&dom, p->dout, p->dtype, ex.B, ex.Tq, p->H, p->D, map_strides(p->do_strides, ex.Tq, ex.packed).s, 128, "dout"))) return rc;
  const void* outs[3] = {p->dq, p->dk, p->dv};
  const int64_t* ostr[3] = {p->dq_strides, p->dk_strides, p->dv_strides};
  for (int t = 0; t < 3; ++t) {
    if ((reinterpret_cast<uintptr_t>(outs[t]) & 15u) != 0) return fail(-3, "gradient pointers must be 16-byte aligned");
    for (int i = ex.packed ? 1 : 0; i < 3; ++i)
      if (ostr[t][i] % 8 != 0) return fail(-3, "gradient strides must be multiples of 8 elements");
  }
  const bool bf = p->dtype == SIGATTN_BF16;
  const bool acc = (p->flags & SIGATTN_ACCURATE) != 0;
  const bool split = (p->flags & SIGATTN_BWD_SPLIT) != 0;
#define SIG_BWD(DD, BF)                                                                   \
  do {                                                                                    \
    if (split) {                                                                          \
      if (acc) return launch_bwd_stream<DD, BF, true>(p, qm, km, vm, dom);                \
      return launch_bwd_stream<DD, BF, false>(p, qm, km, vm, dom);                        \
    }                                                                                     \
    if (acc) return launch_bwd_fused<DD, BF, true>(p, qm, km, vm, dom);                   \
    return launch_bwd_fused<DD, BF, false>(p, qm, km, vm, dom);                           \
  } while (0)
  if (p->D == 64) { if (bf) SIG_BWD(64, true); else SIG_BWD(64, false); }
  else            { if (bf) SIG_BWD(128, true); else SIG_BWD(128, false); }
#undef SIG_BWD
  return fail(-2, "unreachable");
}

int sigattn_bwd_static_scratch(const SigAttnParams* p) {
  g_err[0] = 0;
  int rc = check_common(p, true);
  if (rc < 0) return rc;
  if (rc == 1) return 0;
  const Extents ex = extents(p);
  const unsigned long long elems = (unsigned long long)ex.B * (unsigned long long)ex.Tq * (unsigned long long)p->H *
                                   (unsigned long long)p->D;
  // float32 tensors run the exact kernels, which use no accumulator: no limit applies to them
  if (p->dtype == SIGATTN_FP32) return sigattn_bwd(p);
  if (elems > SIGATTN_STATIC_SCRATCH_ELEMS)
    return fail(-4, "problem too large for the built-in scratch: B*Tq*H*D = %llu elements, limit %u; "
                    "use sigattn_bwd with a caller-provided workspace", elems, (unsigned)SIGATTN_STATIC_SCRATCH_ELEMS);
  float* scratch = nullptr;
  {
    DeviceGuard g;  // makes p->device current for the address lookup
    SIG_CUDA(g.enter(p->device));
    if ((rc = static_scratch_ptr(p->device, &scratch))) return rc;
  }
  // Same path as sigattn_bwd from here on; it zero-fills the accumulator on p->stream first.
  SigAttnParams q = *p;
  q.flags &= ~(uint32_t)SIGATTN_BWD_SPLIT;  // the kernel that accumulates dQ in scratch memory
  q.workspace = scratch;
  q.workspace_bytes = (size_t)SIGATTN_STATIC_SCRATCH_ELEMS * sizeof(float);
  return sigattn_bwd(&q);
}

}  // extern "C"
