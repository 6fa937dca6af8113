// Entry points shared by the attention kernels: workspace sizing and the dense
// form of the reference's pace::attention operands (csrc/ops/attention.cpp:18-97).
#include "common.cuh"

namespace pace {
int run_decode(const KVView& kv, int batch, int n_q_heads, const void* q, int64_t q_sb, int64_t q_sh, void* out,
               int64_t o_sb, int64_t o_sh, const int32_t* kv_start, float scale, void* workspace,
               uint64_t workspace_bytes, cudaStream_t stream);
uint64_t decode_workspace_bytes(int batch, int n_q_heads, int n_kv_heads, int head_dim);
}  // namespace pace

using namespace pace;

extern "C" uint64_t pace_attn_workspace_bytes(int32_t batch, int32_t n_q_heads, int32_t n_kv_heads,
                                              int32_t head_dim, int32_t q_len) {
  (void)q_len;
  if (batch <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0) return 0;
  return decode_workspace_bytes(batch, n_q_heads, n_kv_heads, head_dim);
}

// (multi-token kernels land in attn_mma.cu)
#ifndef PACE_HAVE_MMA
extern "C" int pace_attn_verify(const pace_attn_args_t*, void*) { return PACE_ERR_UNSUPPORTED; }
extern "C" int pace_attn_prefill(const pace_attn_args_t*, void*) { return PACE_ERR_UNSUPPORTED; }
extern "C" int pace_attention_dense(const void*, const void*, const void*, const void*, int32_t, int32_t, void*,
                                    int32_t, int32_t, int32_t, int32_t, int32_t, int32_t, void*, uint64_t, void*) {
  return PACE_ERR_UNSUPPORTED;
}
#endif
