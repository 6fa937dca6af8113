// Shared device/host helpers for the sm_100a KV-cache kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <stdint.h>

#include "pace_b200.h"

namespace pace {

// ---------------------------------------------------------------------------
// Error plumbing (host)
// ---------------------------------------------------------------------------
void set_cuda_error(cudaError_t e, const char* where);

// What the library's newest launch on a stream was (host-side note, kept per stream and device).
// Attention launches let the kernel behind them start early (programmatic dependent launch); the
// note is how a later entry point on the same stream learns what it may overlap with:
//   * an append asks whether the attention launch in front shares its workspace with the launch
//     behind the append (then the append holds its own completion until that launch is done), and
//     whether that launch reads the very layer (or q buffer) the append is about to write (then the
//     append is launched as an ordinary, fully ordered kernel);
//   * a decode launch asks whether anything since the newest attention launch wrote pool state; if
//     not, it may stream K/V ahead of its wait for the kernel in front.
// A stream nobody noted counts as "uses the workspace, wrote the pool".
struct StreamNote {
  cudaStream_t stream;
  int device;
  bool uses_workspace;   // newest attention launch: units may be cut, partials meet in the workspace
  bool pool_written;     // a pool-writing kernel was launched after the newest attention launch
  const void* pages;     // newest attention launch: pool it reads (pages pointer), layer, q buffer
  int layer;
  const void* q;
};
void note_attention_launch(cudaStream_t stream, bool uses_workspace, const void* pages, int layer, const void* q);
void note_pool_write(cudaStream_t stream);
StreamNote stream_note(cudaStream_t stream);
inline bool front_attention_uses_workspace(cudaStream_t stream) { return stream_note(stream).uses_workspace; }

#define PACE_CUDA_TRY(expr)                         \
  do {                                              \
    cudaError_t _e = (expr);                        \
    if (_e != cudaSuccess) {                        \
      ::pace::set_cuda_error(_e, #expr);            \
      return PACE_ERR_CUDA;                         \
    }                                               \
  } while (0)

#define PACE_LAUNCH_CHECK(name)                     \
  do {                                              \
    cudaError_t _e = cudaGetLastError();            \
    if (_e != cudaSuccess) {                        \
      ::pace::set_cuda_error(_e, name);             \
      return PACE_ERR_CUDA;                         \
    }                                               \
  } while (0)

// ---------------------------------------------------------------------------
// What a kernel needs to find K/V rows.  Covers the paged pool (block table,
// per-slot lengths) and a dense [B][Hkv][L][D] tensor (identity table, one
// "page" of L tokens per batch row).
// ---------------------------------------------------------------------------
struct KVView {
  const __nv_bfloat16* k;       // base of this layer's K pages
  const __nv_bfloat16* v;       // base of this layer's V pages
  const int32_t* block_table;   // [max_seqs][max_pages_per_seq] or nullptr (page = slot)
  const int32_t* seq_ids;       // [batch] or nullptr (slot = slot_base + batch index)
  int32_t slot_base;            // first slot of a launch that covers a slice of an unlisted batch
  const int32_t* seq_len;       // this layer's [max_seqs] lengths or nullptr (use fixed_len)
  int32_t* status;              // sticky device status word or nullptr
  int32_t fixed_len;
  int32_t page_tokens;
  int32_t n_kv_heads;
  int32_t head_dim;
  int32_t max_pages_per_seq;
  int32_t max_seqs;
  int32_t n_pages;
};

inline KVView make_view(const pace_kv_pool_t* p, int layer, const int32_t* seq_ids) {
  KVView v;
  const size_t page_elems = (size_t)p->n_kv_heads * p->page_tokens * p->head_dim;
  const size_t region = page_elems * (size_t)p->n_pages;
  const __nv_bfloat16* base = (const __nv_bfloat16*)p->pages;
  v.k = base + ((size_t)layer * 2 + 0) * region;
  v.v = base + ((size_t)layer * 2 + 1) * region;
  v.block_table = p->block_table;
  v.seq_ids = seq_ids;
  v.slot_base = 0;
  v.seq_len = p->seq_len + (size_t)layer * p->max_seqs;
  v.status = p->status;
  v.fixed_len = 0;
  v.page_tokens = p->page_tokens;
  v.n_kv_heads = p->n_kv_heads;
  v.head_dim = p->head_dim;
  v.max_pages_per_seq = p->max_pages_per_seq;
  v.max_seqs = p->max_seqs;
  v.n_pages = p->n_pages;
  return v;
}

#ifdef __CUDACC__

__device__ __forceinline__ void raise_status(int32_t* status, int bits) {
  if (status) atomicOr(status, bits);
}

// slot of batch row b, or -1 when out of range (status raised)
__device__ __forceinline__ int view_slot(const KVView& kv, int b) {
  int s = kv.seq_ids ? kv.seq_ids[b] : b + kv.slot_base;
  if (s < 0 || s >= kv.max_seqs) {
    raise_status(kv.status, PACE_DEV_BAD_INDEX);
    return -1;
  }
  return s;
}
__device__ __forceinline__ int view_len(const KVView& kv, int slot) {
  return kv.seq_len ? kv.seq_len[slot] : kv.fixed_len;
}
// physical page of logical page lp of a slot, or -1
__device__ __forceinline__ int view_page(const KVView& kv, int slot, int lp) {
  if (!kv.block_table) return slot;
  if (lp < 0 || lp >= kv.max_pages_per_seq) return -1;
  int p = kv.block_table[(size_t)slot * kv.max_pages_per_seq + lp];
  if (p < 0 || p >= kv.n_pages) return -1;
  return p;
}
// element offset of row `row` of head h in physical page p
__device__ __forceinline__ size_t view_row_offset(const KVView& kv, int page, int h, int row) {
  return (((size_t)page * kv.n_kv_heads + h) * kv.page_tokens + row) * (size_t)kv.head_dim;
}

// A producer warp's window onto one sequence's block-table row: lane l holds the physical page of
// logical page base + l, and the following window is already on its way.  One coalesced load per
// `step` pages instead of one dependent load per chunk, which would pace the whole pipeline at one
// chunk per memory latency.  All 32 lanes call every method together.
struct PageWindow {
  const int32_t* row;  // nullptr: dense view, every logical page is the slot itself
  int slot, max_pages, n_pages, base, step, cur, nxt;

  __device__ __forceinline__ int load(int l) const {
    if (!row) return slot;
    if (l < 0 || l >= max_pages) return -1;
    const int pg = __ldg(row + l);
    return (pg < 0 || pg >= n_pages) ? -1 : pg;
  }
  // step: how far the window moves at a time (a multiple of the pages one chunk spans, <= 32)
  __device__ __forceinline__ void start(const KVView& kv, int slot_, int first_lp, int step_, int lane) {
    row = kv.block_table ? kv.block_table + (size_t)slot_ * kv.max_pages_per_seq : nullptr;
    slot = slot_;
    max_pages = kv.max_pages_per_seq;
    n_pages = kv.n_pages;
    base = first_lp;
    step = step_;
    cur = load(base + lane);
    nxt = load(base + step + lane);
  }
  // physical page of logical page `lp` (may differ per lane); lp_first is the chunk's first page (uniform)
  __device__ __forceinline__ int get(int lp, int lp_first, int lane) {
    while (lp_first >= base + step) {
      base += step;
      cur = nxt;
      nxt = load(base + step + lane);
    }
    return __shfl_sync(0xffffffffu, cur, (lp - base) & 31);
  }
};

// ---------------------------------------------------------------------------
// mbarrier + bulk-copy (TMA) wrappers.  Every wait is bounded.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// make the initialised barriers visible to the async (TMA) proxy
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One potentially-blocking probe.  The suspend-time hint lets the hardware park the warp until the
// phase completes (or the hint runs out) instead of having it spin: a spinning warp keeps taking
// issue slots from the warps of its scheduler that have work.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"((uint32_t)1000)
      : "memory");
  return ok != 0;
}
// One non-blocking probe.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: true when the phase completed, false when it gave up (after about a quarter of a
// second, or `slow_iters` sleeping probes).  `abort` is a flag in the CTA's shared memory: the first
// role of a CTA whose wait runs out raises it, and every other wait of the CTA that is already
// sleeping returns at once instead of sitting out its own quarter second.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort = nullptr,
                                          int slow_iters = 1 << 18) {
  for (int i = 0; i < 64; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  for (int i = 0; i < slow_iters; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (abort && *abort) return false;
    __nanosleep(64);
  }
  if (abort) *abort = 1;
  return false;
}
// The pool's sticky status word, read without waiting for it: the load is issued here, the thread only
// stalls where it first uses the value (pool_gave_up below).  null -> 0.
__device__ __forceinline__ int load_status_word(const int32_t* status) {
  int v = 0;
  if (status) asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(status));
  return v;
}
// True when the word says that an earlier launch ran out of patience: the launches behind it do
// nothing (and return at once) until the host has cleared the word.
__device__ __forceinline__ bool pool_gave_up(int status_word) { return (status_word & PACE_DEV_WAIT_TIMEOUT) != 0; }
// ---- op timing behind PACE_LOG_LEVEL=profile (host side) ----
// Stands where the reference wraps its operators in PROFILE_PACE_FUNCTION (csrc/core/logging.h:144-212,
// use at csrc/ops/attention.cpp:24): one line "pace::<name>,<info>,<milliseconds>" per call.  Here the
// time is the device time between two CUDA events recorded around the entry point's launches; lines are
// written when the events have completed (the next profiled call, pace_profile_flush or process exit),
// never by waiting inside the call.  Calls made during a stream capture are not timed.
bool profile_enabled();
void profile_begin(const char* name, cudaStream_t stream, cudaEvent_t* e0);
void profile_end(const char* name, const char* info, cudaStream_t stream, cudaEvent_t e0);
struct OpTimer {
  const char* name;
  cudaStream_t stream;
  cudaEvent_t e0 = nullptr;
  char info[96];
  bool on;
  OpTimer(const char* n, void* s) : name(n), stream((cudaStream_t)s), on(profile_enabled()) {
    info[0] = 0;
    if (on) profile_begin(name, stream, &e0);
  }
  ~OpTimer() {
    if (on && e0) profile_end(name, info, stream, e0);
  }
};
#define PACE_PROFILE(name, stream, ...)                                       \
  pace::OpTimer pace_op_timer_(name, stream);                                 \
  if (pace_op_timer_.on) snprintf(pace_op_timer_.info, sizeof(pace_op_timer_.info), __VA_ARGS__)

// global -> shared bulk copy through the TMA unit, completion on an mbarrier.
// Both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// bf16 pair (packed in a 32-bit word, low element first) -> two floats
__device__ __forceinline__ float2 bf2_to_f2(uint32_t w) {
  float2 r;
  r.x = __uint_as_float(w << 16);
  r.y = __uint_as_float(w & 0xffff0000u);
  return r;
}
__device__ __forceinline__ uint32_t f2_to_bf2(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#endif  // __CUDACC__

constexpr float kLog2e = 1.4426950408889634f;
// head of every attention workspace: int32 arrival counters, zero between launches
constexpr uint64_t kWorkspaceCounterBytes = 256 * 1024;

}  // namespace pace
