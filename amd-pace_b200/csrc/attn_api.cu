// Entry points shared by the attention kernels: workspace sizing and the choice of
// decode kernel.
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace pace {
int decode_cuda_cores(const pace_attn_args_t* a, void* stream);
int run_mma_paged(const pace_attn_args_t* a, int causal, cudaStream_t stream);
uint64_t decode_workspace_bytes(int batch, int n_q_heads, int n_kv_heads, int head_dim);
uint64_t mma_workspace_bytes(int n_q_heads, int n_kv_heads, int head_dim, int q_len);
}  // namespace pace

namespace pace {
namespace {
struct StreamNote {
  cudaStream_t stream;
  int device;
  bool uses_workspace;
};
std::mutex g_note_mu;
StreamNote g_notes[64];
int g_n_notes = 0, g_next_note = 0;
}  // namespace

void note_attention_launch(cudaStream_t stream, bool uses_workspace) {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(g_note_mu);
  for (int i = 0; i < g_n_notes; ++i)
    if (g_notes[i].stream == stream && g_notes[i].device == dev) {
      g_notes[i].uses_workspace = uses_workspace;
      return;
    }
  // a full table recycles its oldest entry; a stream that lost its note counts as "uses the workspace"
  StreamNote& n = g_notes[g_next_note];
  g_next_note = (g_next_note + 1) % 64;
  if (g_n_notes < 64) ++g_n_notes;
  n.stream = stream;
  n.device = dev;
  n.uses_workspace = uses_workspace;
}

bool front_attention_uses_workspace(cudaStream_t stream) {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(g_note_mu);
  for (int i = 0; i < g_n_notes; ++i)
    if (g_notes[i].stream == stream && g_notes[i].device == dev) return g_notes[i].uses_workspace;
  return true;
}
}  // namespace pace

using namespace pace;

extern "C" uint64_t pace_attn_workspace_bytes(int32_t batch, int32_t n_q_heads, int32_t n_kv_heads,
                                              int32_t head_dim, int32_t q_len) {
  if (batch <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || q_len <= 0) return 0;
  const uint64_t a = decode_workspace_bytes(batch, n_q_heads, n_kv_heads, head_dim);
  const uint64_t b = mma_workspace_bytes(n_q_heads, n_kv_heads, head_dim, q_len);
  return a > b ? a : b;
}

// Decode (one query token).  Two kernels compute it: the CUDA-core kernel streams K/V rows
// through packed fp32 FMAs and costs G * 2 FMAs per cached byte; the tensor-core kernel packs the
// G grouped query heads into one 16-row MMA tile.  PACE_DECODE_IMPL=cuda|mma forces one of them.
extern "C" int pace_attn_decode(const pace_attn_args_t* a, void* stream) {
  if (!a || !a->pool || a->q_len != 1) return PACE_ERR_INVALID;
  const int G = a->pool->n_kv_heads > 0 ? a->n_q_heads / a->pool->n_kv_heads : 0;
  bool use_mma = G >= 4 && G <= 16;
  if (const char* e = getenv("PACE_DECODE_IMPL")) {
    if (!strcmp(e, "cuda")) use_mma = false;
    if (!strcmp(e, "mma") && G <= 16) use_mma = true;
  }
  return use_mma ? run_mma_paged(a, 1, (cudaStream_t)stream) : decode_cuda_cores(a, stream);
}
