// Entry points shared by the attention kernels: workspace sizing and the choice of
// decode kernel.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace pace {
int decode_cuda_cores(const pace_attn_args_t* a, void* stream);
int run_mma_paged(const pace_attn_args_t* a, int causal, cudaStream_t stream);
uint64_t decode_workspace_bytes(int batch, int n_q_heads, int n_kv_heads, int head_dim);
uint64_t mma_workspace_bytes(int n_q_heads, int n_kv_heads, int head_dim, int q_len);
}  // namespace pace

namespace pace {
namespace {
std::mutex g_note_mu;
StreamNote g_notes[64];
int g_n_notes = 0, g_next_note = 0;

// the stream's note, made (as "unknown": workspace in use, pool written) when there is none;
// a full table recycles its oldest entry.  Call with g_note_mu held.
StreamNote& note_of(cudaStream_t stream) {
  int dev = 0;
  cudaGetDevice(&dev);
  for (int i = 0; i < g_n_notes; ++i)
    if (g_notes[i].stream == stream && g_notes[i].device == dev) return g_notes[i];
  StreamNote& n = g_notes[g_next_note];
  g_next_note = (g_next_note + 1) % 64;
  if (g_n_notes < 64) ++g_n_notes;
  n.stream = stream;
  n.device = dev;
  n.uses_workspace = true;
  n.pool_written = true;
  n.pages = nullptr;
  n.layer = -1;
  n.q = nullptr;
  return n;
}
}  // namespace

void note_attention_launch(cudaStream_t stream, bool uses_workspace, const void* pages, int layer, const void* q) {
  std::lock_guard<std::mutex> lk(g_note_mu);
  StreamNote& n = note_of(stream);
  n.uses_workspace = uses_workspace;
  n.pool_written = false;
  n.pages = pages;
  n.layer = layer;
  n.q = q;
}

void note_pool_write(cudaStream_t stream) {
  std::lock_guard<std::mutex> lk(g_note_mu);
  note_of(stream).pool_written = true;
}

StreamNote stream_note(cudaStream_t stream) {
  std::lock_guard<std::mutex> lk(g_note_mu);
  return note_of(stream);
}
}  // namespace pace


// ---- op timing (PACE_LOG_LEVEL=profile) ----
namespace pace {
namespace {
struct PendingOp {
  cudaEvent_t e0, e1;
  int device;
  char name[32];
  char info[96];
};
std::mutex g_prof_mu;
std::vector<PendingOp> g_pending;
bool g_prof_atexit = false;

// writes the lines of the calls whose events have completed; wait = true waits for every one of them
void profile_drain(bool wait) {
  int cur = 0;
  cudaGetDevice(&cur);
  size_t kept = 0;
  for (size_t i = 0; i < g_pending.size(); ++i) {
    PendingOp& op = g_pending[i];
    cudaSetDevice(op.device);
    cudaError_t st = wait ? cudaEventSynchronize(op.e1) : cudaEventQuery(op.e1);
    if (st == cudaErrorNotReady) {
      g_pending[kept++] = op;
      continue;
    }
    float ms = 0.f;
    if (st == cudaSuccess && cudaEventElapsedTime(&ms, op.e0, op.e1) == cudaSuccess)
      fprintf(stderr, "[PACE profile] pace::%s,%s,%.4f\n", op.name, op.info, ms);
    else
      cudaGetLastError();  // (an untimed call is dropped, its error with it)
    cudaEventDestroy(op.e0);
    cudaEventDestroy(op.e1);
  }
  g_pending.resize(kept);
  cudaSetDevice(cur);
}
}  // namespace

bool profile_enabled() {
  static const bool on = [] {
    const char* v = getenv("PACE_LOG_LEVEL");
    return v && (!strcmp(v, "profile") || !strcmp(v, "PROFILE") || !strcmp(v, "Profile"));
  }();
  return on;
}

void profile_begin(const char* name, cudaStream_t stream, cudaEvent_t* e0) {
  (void)name;
  *e0 = nullptr;
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return;  // events recorded into a graph have no times
  }
  if (cudaEventCreate(e0) != cudaSuccess || cudaEventRecord(*e0, stream) != cudaSuccess) {
    cudaGetLastError();
    if (*e0) cudaEventDestroy(*e0);
    *e0 = nullptr;
  }
}

void profile_end(const char* name, const char* info, cudaStream_t stream, cudaEvent_t e0) {
  PendingOp op;
  op.e0 = e0;
  op.e1 = nullptr;
  cudaGetDevice(&op.device);
  if (cudaEventCreate(&op.e1) != cudaSuccess || cudaEventRecord(op.e1, stream) != cudaSuccess) {
    cudaGetLastError();
    cudaEventDestroy(e0);
    if (op.e1) cudaEventDestroy(op.e1);
    return;
  }
  snprintf(op.name, sizeof(op.name), "%s", name);
  snprintf(op.info, sizeof(op.info), "%s", info);
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (!g_prof_atexit) {
    g_prof_atexit = true;
    atexit([] { pace_profile_flush(); });
  }
  g_pending.push_back(op);
  if (g_pending.size() >= 64) profile_drain(false);
}
}  // namespace pace

extern "C" int pace_profile_enabled(void) { return pace::profile_enabled() ? 1 : 0; }

extern "C" int pace_profile_flush(void) {
  std::lock_guard<std::mutex> lk(pace::g_prof_mu);
  const int n = (int)pace::g_pending.size();
  pace::profile_drain(true);
  return n;
}

using namespace pace;

namespace pace {
namespace {
// Two warps wait on a barrier nobody ever arrives on: the first with a limit of `slow_iters` sleeping
// probes, the second with the kernels' usual quarter second.  The first runs out, raises the CTA's
// abort flag and the pool's PACE_DEV_WAIT_TIMEOUT bit; the second sees the flag and returns at once.
__global__ void wait_selftest_kernel(int32_t* status, int slow_iters) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const bool first = threadIdx.x < 32;
  const bool ok = mbar_wait(&bar, 0, &abort_flag, first ? slow_iters : (1 << 18));
  if (!ok && (threadIdx.x & 31) == 0) raise_status(status, PACE_DEV_WAIT_TIMEOUT);
  __syncthreads();
  if (threadIdx.x == 0) mbar_inval(&bar);
}
}  // namespace
}  // namespace pace

extern "C" int pace_selftest_wait_timeout(const pace_kv_pool_t* pool, int32_t limit_us, void* stream) {
  if (!pool || !pool->status || limit_us < 1 || limit_us > 1000000) return PACE_ERR_INVALID;
  wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(pool->status, (int)limit_us);  // about a microsecond per probe
  PACE_LAUNCH_CHECK("wait_selftest_kernel");
  return PACE_OK;
}

extern "C" uint64_t pace_attn_workspace_bytes(int32_t batch, int32_t n_q_heads, int32_t n_kv_heads,
                                              int32_t head_dim, int32_t q_len) {
  if (batch <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || q_len <= 0) return 0;
  const uint64_t a = decode_workspace_bytes(batch, n_q_heads, n_kv_heads, head_dim);
  const uint64_t b = mma_workspace_bytes(n_q_heads, n_kv_heads, head_dim, q_len);
  return a > b ? a : b;
}

// Decode (one query token).  Two kernels compute it: the tensor-core kernel packs the G grouped
// query heads of a KV head into one mma.sync tile (any G); the CUDA-core kernel streams K/V rows
// through packed fp32 FMAs at G * 2 FMAs per cached byte, which is the cheaper form for G of 1 or 2
// (a 16-row tile would be seven eighths padding).  A launch that carries a pending row always takes
// the tensor-core kernel.
extern "C" int pace_attn_decode(const pace_attn_args_t* a, void* stream) {
  if (!a || !a->pool || a->q_len != 1) return PACE_ERR_INVALID;
  if (a->pool->n_kv_heads <= 0 || a->n_q_heads <= 0 || a->n_q_heads % a->pool->n_kv_heads) return PACE_ERR_INVALID;
  const int G = a->n_q_heads / a->pool->n_kv_heads;
  const bool cuda_cores = G <= 2 && !(a->flags & PACE_ATTN_PENDING_ROW);
  PACE_PROFILE("attn_decode", stream, "layer=%d batch=%d heads=%d/%d head_dim=%d", a->layer, a->batch, a->n_q_heads,
               a->pool->n_kv_heads, a->pool->head_dim);
  return cuda_cores ? decode_cuda_cores(a, stream) : run_mma_paged(a, 1, (cudaStream_t)stream);
}
