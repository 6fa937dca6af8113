// Weight-streaming linear layer for decode steps: Y[M, N] = X[M, K] W[N, K]^T with M <= 32 tokens.
//
// Stands where the reference runs its GEMM back ends on the projections and the MLP of a decoder
// layer (pace/ops/backends/tpp.py:19-63, csrc/ops/libxsmm_linear.cpp:225-241): at a decode batch of
// 32 every weight byte is used for 64 flops, so the layer is bound by reading W once from HBM, not by
// arithmetic.  The kernel is built around that stream:
//   * W is seen as chunks of 128 output rows x 128 input columns (32 KB); the sequence of all chunks
//     (row tile major, columns inside) is cut into equal contiguous ranges, one per CTA, whatever N
//     and K are - no wave quantisation, no tile shape to pick per layer;
//   * one producer warp moves chunks (two 128-byte-swizzled TMA boxes each) and the matching 32 x 128
//     slice of X into a shared-memory ring; eight consumer warps own 16 of the chunk's rows each and
//     run mma.sync m16n8k16 (W rows on the 16-row side, tokens on the 8-column side, fp32 accumulate);
//   * W does not depend on the kernel in front on the stream, so as a programmatic dependent the
//     producer fills the ring with W before griddepcontrol.wait and only X waits for that kernel:
//     the layer's first ~200 KB per SM are on the chip when its input arrives;
//   * a row tile cut by a range boundary is summed in an fp32 workspace with 16-byte reductions that
//     nothing waits for; after its last chunk a CTA settles the (at most two) tiles it holds a part of:
//     fence, one add per tile on the tile's chunk counter, and the CTA that completes a count converts
//     the tile to bf16, stores the rows of Y and leaves workspace and counter at zero for the next call.
// Measured (chains of launches inside one CUDA graph, weights larger than L2): the stream itself runs at
// the copy rate, but the three dependent round trips of that settlement (fence, counter, read-back) cost
// 4-6 us after the last chunk, which a 34-50 MB matrix does not hide; the kernel is ahead of the library
// GEMM only at K = 14336.  The form that removes those round trips - a thread-block cluster per row
// tile, K split across its CTAs with X resident in shared memory and the partial sums exchanged through
// distributed shared memory - is not built.
#include <cuda.h>

#include <cstring>
#include <mutex>

#include "common.cuh"

namespace pace {
namespace {

constexpr int kLinRows = 128;    // W rows per chunk (8 consumer warps x 16)
constexpr int kLinTokens = 32;   // X rows
constexpr int kLinWarps = 8;
constexpr int kLinThreads = kLinWarps * 32 + 32;  // + producer warp
constexpr int kLinStages = 5;
constexpr int kLinCols = 128;              // W columns per chunk: 128 (one CTA per SM) or 64 (two)
constexpr int kLinCtasPerSm = kLinCols == 128 ? 1 : 2;
constexpr int kLinEarlyStages = 5;      // ring stages filled with W before the wait for the kernel in front

template <int COLS>
struct LinShape {
  static constexpr int kBoxes = COLS / 64;                   // 128-byte-swizzled boxes of 64 columns
  static constexpr int kStageW = kLinRows * COLS * 2;        // 32 KB / 16 KB
  static constexpr int kStageX = kLinTokens * COLS * 2;      // 8 KB / 4 KB
  static constexpr int kStage = kStageW + kStageX;
  static constexpr size_t kSmem = (size_t)kLinStages * kStage + 2 * kLinStages * 8 + 64;
};

struct LinParams {
  __nv_bfloat16* y;   // [M][N]
  float* ws;          // [N][32] fp32 partial sums (token order inside a row: see ws_pos), zero between calls
  int32_t* counters;  // [N / 128] chunks summed so far per row tile, zero between calls
  int32_t* status;    // optional sticky status word (PACE_DEV_WAIT_TIMEOUT)
  int M, N, K;
  int64_t y_stride;   // elements between rows of Y
};

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tm, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
// Barrier of the consumer warps only.  The unaligned form: the warps reach it from code in which single
// lanes took a branch of their own (the counter update), so nothing may rely on the compiler keeping one
// barrier instruction per warp.
__device__ __forceinline__ void consumer_barrier() {
  __syncwarp();
  asm volatile("barrier.sync 1, %0;" ::"n"(kLinWarps * 32) : "memory");
}
// Position of a token inside a workspace row: the lane that owns column pair qc of the MMA tile keeps its
// eight tokens (8 t + 2 qc + b, t = 0..3, b = 0..1) next to each other, so that a lane's partial sums of
// one feature are two 16-byte reductions.
__device__ __forceinline__ int ws_token(int pos) { return 8 * ((pos >> 1) & 3) + 2 * (pos >> 3) + (pos & 1); }

template <int COLS>
__global__ void __launch_bounds__(kLinThreads, (COLS == 128 ? 1 : 2))
    linear_skinny_kernel(const LinParams p, const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX) {
  using S = LinShape<COLS>;
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* ring = smem;  // [stages] { W: [boxes][128 rows][128 B], X: [boxes][32 rows][128 B] }
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kLinStages * S::kStage);
  uint64_t* empty_bar = full_bar + kLinStages;
  int* misc = reinterpret_cast<int*>(empty_bar + kLinStages);  // [0] abort flag, [1], [2] "this CTA completes the tile"
  volatile int* abort = misc;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int k_chunks = p.K / COLS, n_tiles = p.N / kLinRows;
  const long long total = (long long)k_chunks * n_tiles;
  const int NC = (long long)gridDim.x < total ? (int)gridDim.x : (int)total;
  const int cta = blockIdx.x;
  if (tid == 0) {
    for (int s = 0; s < kLinStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kLinWarps);
    }
    misc[0] = misc[1] = misc[2] = 0;
    fence_mbar_init();
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmW)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmX)) : "memory");
  }
  __syncthreads();
  if (cta >= NC) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    return;
  }
  const long long x0 = total * cta / NC, x1 = total * (cta + 1) / NC;
  const int n_my = (int)(x1 - x0);

  if (warp == kLinWarps) {
    // ================================ producer ================================
    // W chunks first, for as many stages as the ring has: they do not depend on the kernel in front.
    // Then the wait, then the X slices of those stages, then the steady state.
    const int ahead = n_my < kLinStages ? n_my : kLinStages;
    const int early = ahead < kLinEarlyStages ? ahead : kLinEarlyStages;
    auto issue_w = [&](int i) {
      const long long x = x0 + i;
      const int nt = (int)(x / k_chunks), kc = (int)(x - (long long)nt * k_chunks);
      unsigned char* st = ring + (size_t)i * S::kStage;
      mbar_arrive_expect_tx(&full_bar[i], S::kStage);
#pragma unroll
      for (int b = 0; b < S::kBoxes; ++b) tma_load_2d(st + b * kLinRows * 128, &tmW, kc * COLS + 64 * b, nt * kLinRows, &full_bar[i]);
    };
    if (lane == 0)
      for (int i = 0; i < early; ++i) issue_w(i);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (lane == 0) {
      for (int i = 0; i < ahead; ++i) {
        if (i >= early) issue_w(i);
        const int kc = (int)((x0 + i) % k_chunks);
        unsigned char* sx = ring + (size_t)i * S::kStage + S::kStageW;
#pragma unroll
        for (int b = 0; b < S::kBoxes; ++b) tma_load_2d(sx + b * kLinTokens * 128, &tmX, kc * COLS + 64 * b, 0, &full_bar[i]);
      }
      int issued = ahead;
      bool ok = true;
      for (int i = ahead; i < n_my; ++i) {
        const int s = i % kLinStages;
        if (!mbar_wait(&empty_bar[s], ((i / kLinStages) - 1) & 1, abort)) {
          ok = false;
          break;
        }
        const long long x = x0 + i;
        const int nt = (int)(x / k_chunks), kc = (int)(x - (long long)nt * k_chunks);
        unsigned char* st = ring + (size_t)s * S::kStage;
        mbar_arrive_expect_tx(&full_bar[s], S::kStage);
#pragma unroll
        for (int b = 0; b < S::kBoxes; ++b) tma_load_2d(st + b * kLinRows * 128, &tmW, kc * COLS + 64 * b, nt * kLinRows, &full_bar[s]);
#pragma unroll
        for (int b = 0; b < S::kBoxes; ++b)
          tma_load_2d(st + S::kStageW + b * kLinTokens * 128, &tmX, kc * COLS + 64 * b, 0, &full_bar[s]);
        issued = i + 1;
      }
      if (!ok) {
        raise_status(p.status, PACE_DEV_WAIT_TIMEOUT);
        // copies in flight land before the CTA's shared memory is released (these waits are never cut short)
        const int from = issued > kLinStages ? issued - kLinStages : 0;
        for (int k = from; k < issued; ++k) mbar_wait(&full_bar[k % kLinStages], (k / kLinStages) & 1);
      }
    }
    return;
  }

  // ================================= consumers =================================
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int qr = lane >> 2, qc = lane & 3;
  float acc[4][4];
#pragma unroll
  for (int t = 0; t < 4; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
  int seg_chunks = 0;  // chunks accumulated for the current row tile
  // Row tiles this CTA holds only a part of: at most the one its range starts in and the one it ends in.
  int part_nt0 = -1, part_seg0 = 0, part_nt1 = -1, part_seg1 = 0;
  for (int i = 0; i < n_my; ++i) {
    const int s = i % kLinStages;
    if (!mbar_wait(&full_bar[s], (i / kLinStages) & 1, abort)) {
      if (lane == 0) raise_status(p.status, PACE_DEV_WAIT_TIMEOUT);
      break;  // the abort flag is up: every warp leaves its loop and meets the others at the barrier below
    }
    const long long x = x0 + i;
    const int nt = (int)(x / k_chunks), kc = (int)(x - (long long)nt * k_chunks);
    const uint32_t wb = smem_u32(ring + (size_t)s * S::kStage), xb = wb + S::kStageW;
    const int mi = lane >> 3;
    // A: my 16 rows of W, 16 columns per step.  B: all 32 tokens of X at the same columns.
    const int arow = warp * 16 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
    for (int k = 0; k < COLS / 16; ++k) {
      const int cg = k * 2 + (mi >> 1);  // 16-byte column group of the A matrices
      uint32_t a0, a1, a2, a3;
      ldsm4(wb + (cg >> 3) * (kLinRows * 128) + arow * 128 + (((cg & 7) ^ (arow & 7)) << 4), a0, a1, a2, a3);
#pragma unroll
      for (int t2 = 0; t2 < 2; ++t2) {  // tokens 16 t2 .. 16 t2 + 15: matrices (tokens lo, k lo), (lo, hi), (hi, lo), (hi, hi)
        const int brow = t2 * 16 + (mi >> 1) * 8 + (lane & 7);
        const int bg = k * 2 + (mi & 1);
        uint32_t b0, b1, b2, b3;
        ldsm4(xb + (bg >> 3) * (kLinTokens * 128) + brow * 128 + (((bg & 7) ^ (brow & 7)) << 4), b0, b1, b2, b3);
        mma_bf16(acc[2 * t2], a0, a1, a2, a3, b0, b1);
        mma_bf16(acc[2 * t2 + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);
    ++seg_chunks;
    const bool tile_ends = kc == k_chunks - 1 || i == n_my - 1;
    if (!tile_ends) continue;
    // ---- my 16 rows x 32 tokens of this row tile leave the registers ----
    // acc[t][0..1]: row qr, tokens 8 t + 2 qc + {0, 1}; acc[t][2..3]: row qr + 8
    const int f0 = nt * kLinRows + warp * 16 + qr;
    if (seg_chunks == k_chunks) {  // nobody else holds a part of this tile
#pragma unroll
      for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = 8 * t + 2 * qc + (e & 1), f = f0 + (e >> 1) * 8;
          if (tok < p.M) p.y[(size_t)tok * p.y_stride + f] = __float2bfloat16(acc[t][e]);
        }
    } else {
      // partial sums into the workspace: fire and forget, nothing waits here (the stream goes on);
      // the tile's completion is settled once, after this CTA's last chunk
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float* w = p.ws + (size_t)(f0 + 8 * h) * kLinTokens + qc * 8;
        red_add_v4(w, acc[0][2 * h], acc[0][2 * h + 1], acc[1][2 * h], acc[1][2 * h + 1]);
        red_add_v4(w + 4, acc[2][2 * h], acc[2][2 * h + 1], acc[3][2 * h], acc[3][2 * h + 1]);
      }
      if (part_nt0 < 0) {
        part_nt0 = nt;
        part_seg0 = seg_chunks;
      } else {
        part_nt1 = nt;
        part_seg1 = seg_chunks;
      }
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
    seg_chunks = 0;
  }
  // ---- settle the row tiles this CTA holds a part of ----
  __threadfence();     // my reductions are performed before the counter says so
  consumer_barrier();  // ... and so are everybody else's of this CTA
  if (*abort) return;
  if (part_nt0 < 0) return;  // (the same in every consumer thread)
  if (warp == 0 && lane < 2) {
    const int nt = lane == 0 ? part_nt0 : part_nt1, seg = lane == 0 ? part_seg0 : part_seg1;
    if (nt >= 0) {
      const int old = atomicAdd(&p.counters[nt], seg);
      misc[1 + lane] = (old + seg == k_chunks);
    }
  }
  consumer_barrier();
  // A complete tile sits in the workspace as 128 features x 32 tokens; a thread takes half a feature's
  // row.  Both tiles' loads are in flight before anything is stored: one round trip, not two.
  const bool conv0 = misc[1] != 0, conv1 = part_nt1 >= 0 && misc[2] != 0;
  if (!conv0 && !conv1) return;
  __threadfence();
  const int half = tid >> 7;
  float v[2][16];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    if (!(j == 0 ? conv0 : conv1)) continue;
    const int f = (j == 0 ? part_nt0 : part_nt1) * kLinRows + (tid & 127);
    const float4* w4 = reinterpret_cast<const float4*>(p.ws + (size_t)f * kLinTokens + half * 16);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 r = __ldcg(w4 + q);
      v[j][4 * q] = r.x; v[j][4 * q + 1] = r.y; v[j][4 * q + 2] = r.z; v[j][4 * q + 3] = r.w;
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    if (!(j == 0 ? conv0 : conv1)) continue;
    const int nt = j == 0 ? part_nt0 : part_nt1;
    const int f = nt * kLinRows + (tid & 127);
    float4* w4 = reinterpret_cast<float4*>(p.ws + (size_t)f * kLinTokens + half * 16);
#pragma unroll
    for (int q = 0; q < 4; ++q) w4[q] = make_float4(0.f, 0.f, 0.f, 0.f);  // workspace and counter ready for the next call
    if (tid == 0) p.counters[nt] = 0;
#pragma unroll
    for (int q = 0; q < 16; ++q) {
      const int tok = ws_token(half * 16 + q);
      if (tok < p.M) p.y[(size_t)tok * p.y_stride + f] = __float2bfloat16(v[j][q]);
    }
  }
}

typedef CUresult (*EncodeFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn2 encode_fn2() {
  static EncodeFn2 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn2>(ptr);
  });
  return fn;
}

// bf16 matrix [rows][cols] with a row pitch; box = 64 columns x box_rows rows, 128-byte swizzle, zero fill outside
int make_map_2d(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_elems, int box_rows) {
  EncodeFn2 fn = encode_fn2();
  if (!fn) {
    set_cuda_error(cudaErrorNotSupported, "cuTensorMapEncodeTiled entry point");
    return PACE_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch_elems * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled (linear)");
    return PACE_ERR_CUDA;
  }
  return PACE_OK;
}

struct WMapEntry {
  const void* w;
  int64_t n, k, pitch;
  CUtensorMap tm;
};
std::mutex g_wmap_mu;
WMapEntry g_wmaps[512];
int g_n_wmaps = 0, g_next_wmap = 0;

}  // namespace
}  // namespace pace

using namespace pace;


extern "C" uint64_t pace_linear_workspace_bytes(int32_t n_max) {
  if (n_max <= 0) return 0;
  const uint64_t ws = (uint64_t)kLinTokens * (uint64_t)n_max * sizeof(float);
  return ws + ((uint64_t)(n_max / kLinRows) + 1) * sizeof(int32_t) + 256;
}

extern "C" int pace_linear_skinny(const void* x, int64_t x_stride, const void* w, int64_t w_stride, void* y,
                                  int64_t y_stride, int32_t M, int32_t N, int32_t K, void* workspace,
                                  uint64_t workspace_bytes, int32_t* status, void* stream) {
  if (!x || !w || !y || !workspace || M < 1 || N < 1 || K < 1) return PACE_ERR_INVALID;
  if (M > kLinTokens || N % kLinRows || K % kLinCols) return PACE_ERR_UNSUPPORTED;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)workspace & 31) || (x_stride & 7) || (w_stride & 7))
    return PACE_ERR_INVALID;
  if (x_stride < K || w_stride < K || y_stride < N) return PACE_ERR_INVALID;
  if (workspace_bytes < pace_linear_workspace_bytes(N)) return PACE_ERR_INVALID;
  PACE_PROFILE("linear_skinny", stream, "x=[%d,%d] w=[%d,%d]", M, K, N, K);
  CUtensorMap tmW, tmX;
  {
    std::lock_guard<std::mutex> lk(g_wmap_mu);
    const CUtensorMap* hit = nullptr;
    for (int i = 0; i < g_n_wmaps; ++i)
      if (g_wmaps[i].w == w && g_wmaps[i].n == N && g_wmaps[i].k == K && g_wmaps[i].pitch == w_stride) hit = &g_wmaps[i].tm;
    if (hit) {
      tmW = *hit;
    } else {
      const int rc = make_map_2d(&tmW, w, (uint64_t)N, (uint64_t)K, (uint64_t)w_stride, kLinRows);
      if (rc != PACE_OK) return rc;
      WMapEntry& e = g_wmaps[g_next_wmap];
      g_next_wmap = (g_next_wmap + 1) % 512;
      if (g_n_wmaps < 512) ++g_n_wmaps;
      e.w = w; e.n = N; e.k = K; e.pitch = w_stride; e.tm = tmW;
    }
  }
  int rc = make_map_2d(&tmX, x, (uint64_t)M, (uint64_t)K, (uint64_t)x_stride, kLinTokens);
  if (rc != PACE_OK) return rc;
  LinParams p;
  p.y = (__nv_bfloat16*)y;
  p.ws = (float*)workspace;
  p.counters = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + (size_t)kLinTokens * N * sizeof(float));
  p.status = status;
  p.M = M; p.N = N; p.K = K;
  p.y_stride = y_stride;
  int dev = 0, sms = 148;
  PACE_CUDA_TRY(cudaGetDevice(&dev));
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const size_t smem_bytes = LinShape<kLinCols>::kSmem;
  static bool configured[16] = {};
  if (dev >= 16 || !configured[dev]) {
    PACE_CUDA_TRY(cudaFuncSetAttribute(linear_skinny_kernel<kLinCols>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    if (dev < 16) configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(sms * kLinCtasPerSm));
  cfg.blockDim = dim3(kLinThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  PACE_CUDA_TRY(cudaLaunchKernelEx(&cfg, linear_skinny_kernel<kLinCols>, p, tmW, tmX));
  PACE_LAUNCH_CHECK("linear_skinny_kernel");
  return PACE_OK;
}
