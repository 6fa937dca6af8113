// Tensor-core attention over the paged KV pool: short-query verify (PARD), chunked
// prefill, the dense form of the reference op, and GQA decode with the query-head
// group packed into one MMA tile.
//
// Replaces the reference's four-primitive SDPA sequence
// (csrc/ops/kernels/attention_kernels.cpp:218-257) for S >= 1 query tokens: the
// [B,N,S,L] score tensor is never materialised, K/V are read once per query tile.
//
// Shape of the kernel:
//   * the query rows of one (sequence, kv head) are the S tokens x G grouped heads,
//     row r = s * G + g, cut into tiles of 16 * MT rows;
//   * persistent grid, one CTA per SM; the global sequence of K/V chunks of all
//     (sequence, query tile, kv head) units is cut into equal contiguous ranges;
//   * one producer warp: tiled TMA copies (cp.async.bulk.tensor, 128-byte swizzle)
//     of K and V pages into a shared-memory ring, per-row bulk copies of the Q tile;
//   * eight consumer warps arranged MT x NS: warp (mt, ns) owns 16 query rows and
//     the ns-th slice of every chunk's tokens; S = Q K^T and O += P V are
//     mma.sync m16n8k16 (bf16 in, fp32 accumulate), online softmax in registers;
//   * the NS slices of a tile are merged through shared memory; a unit cut by a
//     range boundary leaves an fp32 partial in the workspace and the last CTA to
//     arrive merges (no CTA waits on another).
#include <cuda.h>

#include <climits>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace pace {
namespace {

// Threads of a CTA with nw consumer warps: + producer warp + epilogue warp (tcgen05 variant: + producer
// warp + two MMA issuer warps).  Eight consumer warps and one CTA per SM, or - decode only - four and
// two CTAs per SM, so that CTAs of the next launch on the stream move in beside CTAs of this one.
__host__ __device__ constexpr int threads_of(bool umma, int nw = 8) { return nw * 32 + (umma ? 128 : 64); }
constexpr int kChunk = 64;
constexpr int kMaxStagesM = 8;
constexpr int kMaxItems = 1024;

struct MetaM {  // one 64-byte record per ring stage, written by the producer
  int rows, tok0, flags, kvs;
  int b, h, r_lo, R;
  int kv_len, S, mode, parts;
  int first_cta, first_slot, unit, pad;  // pad: chunks of the unit part (on its first chunk's record)
};
static_assert(sizeof(MetaM) == 64, "MetaM is one 64-byte line");

struct MmaParams {
  KVView kv;
  int c3_k, c3_v;  // 4th tensor-map coordinate of the K and of the V region
  const __nv_bfloat16* q;
  int64_t q_sb, q_sh, q_ss;
  __nv_bfloat16* out;
  int64_t o_sb, o_sh, o_ss;
  const int32_t* kv_start;
  const int32_t* q_lens;
  int batch, q_len, G, n_qt, causal;
  int whole_units;  // never cut a unit across CTAs (no workspace traffic)
  float scale_log2;
  float* parts;
  int32_t* unit_count;
  int chunk_tokens, pages_per_chunk, chunks_per_page, box_rows, n_stages, live_max;
  const void* mask;  // additive [B,1,mask_rows,L] or null
  int mask_fp32, mask_rows;
  int64_t mask_sb;
  // decode with a pending row: key number kv_len of every (sequence, kv head), not in the pool yet
  const __nv_bfloat16* k_pend;
  const __nv_bfloat16* v_pend;
  int64_t pend_sb, pend_sh;
  int early_kv;  // whole-unit decode: K/V copies may leave ahead of the wait for the kernel in front
  int sub_boxes;  // 64-token pages: a unit's partly filled last page is fetched in 16-row boxes (tmS)
};

__device__ __forceinline__ int chunks_of_m(const MmaParams& p, int len) {
  if (len <= 0) return 0;
  if (p.pages_per_chunk > 0) return (len + p.chunk_tokens - 1) / p.chunk_tokens;
  const int P = p.kv.page_tokens;
  const int full = len / P, rem = len - full * P;
  return full * p.chunks_per_page + (rem + kChunk - 1) / kChunk;
}

template <int CTHR>
__device__ __forceinline__ void csync() { asm volatile("bar.sync 1, %0;" ::"n"(CTHR) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// (m16n8k8: for consumer slices of eight keys, a form no current instantiation takes)
__device__ __forceinline__ void mma1688(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(b0));
}
// 8x8 b16 matrix held in fragment layout (thread: row lane / 4, columns 2 * (lane % 4) + {0, 1}) -> its transpose
__device__ __forceinline__ uint32_t movmatrix_t(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
// tiled TMA load of one box into this CTA, completion on an mbarrier
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* tm, int c0, int c1, int c2, int c3,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];" ::"r"(smem_u32(smem_dst)),
      "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// The same copy with an L2 eviction policy: decode and verify (one query tile per sequence and KV head)
// stream every K/V byte once per launch, and marked
// evict-first the stream leaves the small things every launch starts with (block table, lengths, query
// rows) in L2 instead of pushing them out.
__device__ __forceinline__ void tma_load_4d_hint(void* smem_dst, const CUtensorMap* tm, int c0, int c1, int c2, int c3,
                                                 uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, "
      "%4, %5, %6}], [%2], %7;" ::"r"(smem_u32(smem_dst)),
      "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

// Shared-memory carve-up, computed identically on host and device.
struct SmemPlan {
  int ring, metas, qbuf, mg, res, bars, misc, per_b, prefix, total;
  int res_slot_bytes, n_res, mg_stride;
};
// (umma: the tcgen05 variant keeps its Q tile in tensor memory and needs neither the padded Q rows,
// the merge buffer nor the result slots)
__host__ __device__ inline SmemPlan plan_smem(int D, int MT, int NS, int n_stages, int live_max, int batch,
                                              int n_items, bool umma = false) {
  SmemPlan s;
  const int MR = 16 * MT, QS = D * 2 + 16;
  int off = 0;
  auto take = [&](int bytes, int align) {
    off = (off + align - 1) / align * align;
    const int o = off;
    off += bytes;
    return o;
  };
  s.ring = take(n_stages * 2 * kChunk * D * 2, 1024);
  // (mma.sync kernels: only the live rows are ever written; a fragment load of the padding rows of the
  // last 8-row group and beyond reads whatever follows in shared memory, which no live row depends on)
  const int q_rows = MR < ((live_max + 7) & ~7) ? MR : ((live_max + 7) & ~7);
  // (the tcgen05 variant keeps its Q tile in tensor memory; with two tiles per unit the second one's is here)
  s.qbuf = umma ? (MT == 16 ? take(128 * D * 2, 1024) : take(16, 16)) : take(q_rows * QS, 128);
  s.mg_stride = D + 8;  // floats; the pad spreads the rows of a fragment over the banks
  s.mg = take(umma ? 16 : (NS > 1 ? NS * live_max * (s.mg_stride + 2) * 4 : 16), 16);
  s.n_res = live_max <= 64 ? 2 : 1;
  s.res_slot_bytes = (live_max * (D + 2) * 4 + 64 + 15) / 16 * 16;
  s.res = take(umma ? 16 : s.n_res * s.res_slot_bytes, 16);
  s.metas = take(n_stages * (int)sizeof(MetaM), 64);
  s.bars = take((2 * kMaxStagesM + 1 + 4 + (umma ? 20 : 0)) * 8, 8);
  s.misc = take(8 * 4, 4);
  s.per_b = take(batch * 4 * 4, 4);
  s.prefix = take((n_items + 1) * 4, 4);
  s.total = (off + 15) / 16 * 16;
  return s;
}

constexpr int kHalfSmemBudget = 113 * 1024;  // two CTAs per SM: 228 KB less the 1 KB the system keeps per CTA

struct ResMeta {  // trails each result slot
  int b, h, r_lo, live, mode, parts, first_cta, first_slot, unit, last_part, pad[6];
};
static_assert(sizeof(ResMeta) == 64, "ResMeta is one 64-byte line");

}  // namespace
}  // namespace pace
#include "attn_umma.cuh"
namespace pace {
namespace {

// Takes one finished unit part from its shared-memory result slot to global memory: the output
// rows (mode 0), or an fp32 partial plus the arrival count and, for the last arriver, the merge
// of all partials.  Run by a group of NTHR threads: one warp (WARP) or the eight consumer warps.
template <int D, int MR, int NTHR, bool WARP>
__device__ __forceinline__ void publish_part(const MmaParams& p, const ResMeta& rm, const float* rnum, const float* rM,
                                             const float* rden, int t, int cta, int* flag) {
  constexpr int REC = MR * (D + 2);
  const int G = p.G, live = rm.live;
  auto group_sync = [&]() {
    if (WARP) __syncwarp(); else csync<NTHR>();
  };
  if (rm.mode == 0) {
    for (int oi = t * 2; oi < live * D; oi += NTHR * 2) {
      const int row = oi / D, d = oi - row * D;
      const float den = rden[row];
      const float inv = den > 0.f ? 1.0f / den : 0.f;
      const int r = rm.r_lo + row, sq = r / G, g = r - sq * G;
      *reinterpret_cast<uint32_t*>(p.out + (size_t)rm.b * p.o_sb + (size_t)(rm.h * G + g) * p.o_sh +
                                   (size_t)sq * p.o_ss + d) = f2_to_bf2(rnum[oi] * inv, rnum[oi + 1] * inv);
    }
    return;
  }
  // Fast path for the CTA's last part (the consumer warps' call): it is usually the last of its unit
  // to arrive, and then its own result never needs to leave shared memory.  One acquiring load of the
  // arrival count decides; no other CTA can arrive once parts - 1 have.
  int own = -1;  // index of this CTA's part when it is merged straight from shared memory
  if (!WARP) {
    if (t == 0) {
      int seen;
      asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.unit_count + rm.unit) : "memory");
      *flag = (seen == rm.parts - 1);
      if (seen == rm.parts - 1) p.unit_count[rm.unit] = 0;  // ready for the next launch
    }
    csync<NTHR>();
    if (*flag) own = cta - rm.first_cta;
    csync<NTHR>();  // flag is rewritten below
  }
  float* rec = p.parts + ((size_t)cta * 2 + (rm.mode == 2 ? 1 : 0)) * REC;
  if (own < 0) {
  for (int oi = t * 2; oi < live * D; oi += NTHR * 2)
    *reinterpret_cast<float2*>(rec + oi) = *reinterpret_cast<const float2*>(rnum + oi);
  for (int row = t; row < live; row += NTHR) {
    rec[MR * D + row] = rM[row];
    rec[MR * D + MR + row] = rden[row];
  }
  __threadfence();
  group_sync();
  int is_last = 0;
  if (t == 0) {
    const int old = atomicAdd(&p.unit_count[rm.unit], 1);
    is_last = (old == rm.parts - 1);
    if (is_last) p.unit_count[rm.unit] = 0;  // ready for the next launch
    if (!WARP) *flag = is_last;
  }
  if (WARP) {
    is_last = __shfl_sync(0xffffffffu, is_last, 0);
  } else {
    csync<NTHR>();
    is_last = *flag;
  }
  if (!is_last) return;
  __threadfence();
  }  // own < 0
  for (int oi = t * 2; oi < live * D; oi += NTHR * 2) {
    const int row = oi / D, d = oi - row * D;
    float M = -INFINITY, n0 = 0.f, n1 = 0.f, den = 0.f;
    for (int c0 = 0; c0 < rm.parts; c0 += 4) {  // four partials' loads in flight at a time
      float mc[4], dc[4];
      float2 nn[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = c0 + k;
        mc[k] = -INFINITY;
        dc[k] = 0.f;
        nn[k] = make_float2(0.f, 0.f);
        if (c == own) {
          mc[k] = rM[row];
          dc[k] = rden[row];
          nn[k] = *reinterpret_cast<const float2*>(rnum + oi);
        } else if (c < rm.parts) {
          const float* r = p.parts + ((size_t)(rm.first_cta + c) * 2 + (c == 0 ? rm.first_slot : 0)) * REC;
          mc[k] = __ldcg(r + MR * D + row);
          dc[k] = __ldcg(r + MR * D + MR + row);
          nn[k] = __ldcg(reinterpret_cast<const float2*>(r + oi));
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float Mn = fmaxf(M, mc[k]);
        if (Mn != -INFINITY) {
          const float a = (M == -INFINITY) ? 0.f : fast_exp2(M - Mn);
          const float f = (mc[k] == -INFINITY) ? 0.f : fast_exp2(mc[k] - Mn);
          n0 = n0 * a + nn[k].x * f;
          n1 = n1 * a + nn[k].y * f;
          den = den * a + dc[k] * f;
          M = Mn;
        }
      }
    }
    const float inv = den > 0.f ? 1.0f / den : 0.f;
    const int rr = rm.r_lo + row, sq = rr / G, g = rr - sq * G;
    *reinterpret_cast<uint32_t*>(p.out + (size_t)rm.b * p.o_sb + (size_t)(rm.h * G + g) * p.o_sh + (size_t)sq * p.o_ss +
                                 d) = f2_to_bf2(n0 * inv, n1 * inv);
  }
}

// One warp stores the pending K and V row of (sequence b, kv head h) in their slot of the pool: row
// number seq_len of the sequence, i.e. the first unused row of its last page (or the first row of the
// page behind it, which the step's reservation has made sure of).  seq_len is left alone.  Lanes
// 0..15 move the K row, 16..31 the V row, 16 bytes each.  Returns false on a bad slot or page.
template <int D>
__device__ __forceinline__ bool store_pending_row(const MmaParams& p, int b, int h, int lane) {
  const int slot = view_slot(p.kv, b);
  if (slot < 0) return false;
  const int len = view_len(p.kv, slot), P = p.kv.page_tokens;
  const int lp = len / P;
  const int pg = view_page(p.kv, slot, lp);
  if (pg < 0) return false;
  const int half = lane >> 4, l16 = lane & 15;
  if (l16 < D / 8) {
    const __nv_bfloat16* src = (half ? p.v_pend : p.k_pend) + (size_t)b * p.pend_sb + (size_t)h * p.pend_sh;
    __nv_bfloat16* dst = const_cast<__nv_bfloat16*>(half ? p.kv.v : p.kv.k) + view_row_offset(p.kv, pg, h, len - lp * P);
    reinterpret_cast<uint4*>(dst)[l16] = __ldcg(reinterpret_cast<const uint4*>(src) + l16);
  }
  return true;
}
// the row stores above (generic proxy) are performed, then ordered before async-proxy reads (the TMA
// copy of that page)
__device__ __forceinline__ void fence_proxy_async_all() {
  __threadfence();
  asm volatile("fence.proxy.async;" ::: "memory");
}

template <int D, int MT, int NS, bool UMMA = false>
__global__ void __launch_bounds__(threads_of(UMMA, UMMA ? 8 : MT * NS), (!UMMA && MT * NS == 4) ? 2 : 1)
    attn_mma_kernel(const MmaParams p, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const __grid_constant__ CUtensorMap tmS) {
  constexpr int NW = UMMA ? 8 : MT * NS;  // consumer warps (the tcgen05 variant: eight softmax warps whatever the tile)
  constexpr bool WIDE = UMMA && MT == 16;  // 256 query rows per unit: two 128-row tiles share every K/V chunk
  constexpr int CTHR = NW * 32;
  static_assert(NW == 8 || (NW == 4 && MT == 1 && !UMMA), "eight consumer warps, or four in the two-per-SM decode form");
  constexpr int NTHR = threads_of(UMMA, NW);
  static_assert(!UMMA || ((MT == 8 || MT == 16) && NS == 1), "the tcgen05 variant works on 128-row tiles, one or two per unit");
  // How the NS warps of a row tile share the key stream: DG groups of SL warps; chunk i goes to group
  // i % DG, whose warps cut its keys into SL slices.  Verify tiles (MT, NS >= 2): DG = NS, whole chunks
  // are dealt round-robin to the warps, so NS chunks are in flight in the tensor pipe at a time and a
  // warp's MMA chains have 8 independent tiles to overlap.  Decode (MT == 1) with eight warps: two groups
  // of four warps, 16 keys per warp - one group works on chunk i while the other already has chunk i + 1
  // (measured on batch 32, 600 cached tokens: 22.6 us with one group of eight slices, 21.5 us with two
  // groups, 22.6 us with four, 24.5 us with whole chunks per warp).  Decode with four warps (two CTAs per
  // SM, each with its own producer warp and a three-stage ring): one group, 16 keys per warp; the two
  // CTAs of an SM are the two groups, and they drift apart instead of marching in step - 19.3 us
  // (1=2, two groups of two warps with 32 keys each, holds two of the three ring
  // stages at a time: 19.1 us where one group takes 18.0 us).
  constexpr int DG = (MT >= 2 && NS >= 2) ? NS : (MT == 1 ? (NS == 4 ? 1 : 2) : 1);
  constexpr int SL = NS / DG;
  constexpr int TW = kChunk / SL;  // keys of a chunk one warp works on
  constexpr int NT = TW / 8;                              // score n-tiles per warp
  constexpr int KS = D / 16;       // k-steps of Q K^T
  constexpr int ON = D / 8;        // output n-tiles
  constexpr int HALVES = D / 64;   // 64-element (128-byte) column blocks of a K/V row
  constexpr int MR = 16 * MT;      // query rows per tile
  constexpr int QS = D * 2 + 16;   // padded Q row stride in shared memory (bytes)
  constexpr int KVB = kChunk * D * 2;  // bytes of one K (or V) chunk slot
  constexpr int HALF_B = kChunk * 128;
  constexpr int STAGE = 2 * KVB;

  extern __shared__ __align__(1024) unsigned char smem[];
  const int n_stages = p.n_stages;
  const int n_items = p.batch * p.n_qt;
  // pend: every sequence has one more key than the pool says, whose row this launch first stores in
  // its slot of the sequence's last page (position seq_len; seq_len itself is left alone)
  const bool pend = !UMMA && p.k_pend != nullptr;
  const SmemPlan sp = plan_smem(D, MT, NS, n_stages, p.live_max, p.batch, n_items, UMMA);
  unsigned char* ring = smem + sp.ring;  // [n_stages][K | V]
  MetaM* metas = reinterpret_cast<MetaM*>(smem + sp.metas);
  unsigned char* qbuf = smem + sp.qbuf;
  float* mg_o = reinterpret_cast<float*>(smem + sp.mg);          // [NS][live_max][mg_stride]
  float* mg_m = mg_o + NS * p.live_max * sp.mg_stride;           // [NS][live_max]
  float* mg_l = mg_m + NS * p.live_max;                          // [NS][live_max]
  unsigned char* res = smem + sp.res;                            // [n_res] { num[live][D], M[live], den[live], ResMeta }
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + sp.bars);
  uint64_t* empty_bar = full_bar + kMaxStagesM;
  uint64_t* q_empty = empty_bar + kMaxStagesM;
  uint64_t* res_full = q_empty + 1;   // [2]
  uint64_t* res_empty = res_full + 2; // [2]
  uint64_t* umma_bars = res_empty + 2; // [20], tcgen05 variant only
  int* misc = reinterpret_cast<int*>(smem + sp.misc);
  volatile int* abort = misc + 4;  // raised by the first role whose wait runs out (and from the start on a pool that has given up)
  int* sb_slot = reinterpret_cast<int*>(smem + sp.per_b);
  int* sb_len = sb_slot + p.batch;
  int* sb_kvs = sb_len + p.batch;
  int* sb_S = sb_kvs + p.batch;
  int* prefix = reinterpret_cast<int*>(smem + sp.prefix);  // [items + 1]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int Hkv = p.kv.n_kv_heads, P = p.kv.page_tokens, G = p.G;

  // ---- prologue, part 1: what depends on nothing an earlier kernel wrote.  Barrier set-up and the
  // zero fill of the V slots (rows no copy ever writes are multiplied by p = 0 and must not hold NaN
  // patterns).  When the kernel is launched as a programmatic dependent this part runs while the
  // kernel in front of it on the stream drains; griddepcontrol.wait then holds until that kernel has
  // completed and its writes (the appended rows, the lengths) are visible. ----
  // one barrier per thread of the last warp (its lanes have no sequences to look up in small batches)
  if (tid == NW * 32) {
    // the producer's first tiled copy would otherwise wait for its 128-byte descriptor to arrive
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmK)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmV)) : "memory");
    if (p.sub_boxes) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmS)) : "memory");
  }
  if (tid >= NTHR - 32) {
    const int k = tid - (NTHR - 32);
    if (k < n_stages) mbar_init(&full_bar[k], 1);
    else if (k < 2 * n_stages) mbar_init(&empty_bar[k - n_stages], UMMA ? (WIDE ? 2 : 1) : NW);  // (wide: one commit per group's PV)
    else if (k == 2 * n_stages) mbar_init(q_empty, NW);
    else if (k < 2 * n_stages + 3) mbar_init(&res_full[k - 2 * n_stages - 1], NW);
    else if (k < 2 * n_stages + 5) mbar_init(&res_empty[k - 2 * n_stages - 3], 1);
    if (k == 30) {
      misc[2] = 0;  // longest unit, in chunks (a maximum over the items, taken below)
      misc[4] = 0;  // the CTA's abort flag
    }
    if (UMMA && k == 31) {
      // s_full[2] (+2 unused), p_full[2] and s_free[2] (one arrival per warp of the group), o_full[2],
      // q_ready, drain[2], pub (every softmax thread), xch (one arrival per softmax warp, like q_ready)
      for (int j = 0; j < 19; ++j)
        mbar_init(&umma_bars[j],
                  (j >= 4 && j < 8) ? 4 : (j == 10 || j == 14) ? 8 : (j == 13 ? kUmmaSoftmaxThreads : 1));
    }
    fence_mbar_init();
  }
  for (int s = 0; s < n_stages; ++s) {
    // (tcgen05 variant: the ring is [K column block 0 of every stage][K column block 1 ...][V of every
    // stage], so that the K rows of two consecutive stages are contiguous and one MMA can span both)
    uint4* z = reinterpret_cast<uint4*>(UMMA ? ring + (size_t)n_stages * KVB + (size_t)s * KVB
                                             : ring + (size_t)s * STAGE + KVB);
    for (int i = tid; i < KVB / 16; i += NTHR) z[i] = make_uint4(0, 0, 0, 0);
  }
  // Short prologue (decode told to keep units whole, PACE_ATTN_WHOLE_UNITS): the CTA's units are known
  // from its index alone, so the producer warp needs nobody else - it looks up its own few sequences
  // and starts streaming while the general prologue below would still be counting every sequence's
  // chunks behind three CTA-wide barriers (about 2 us of a 19 us launch).  The consumers learn where
  // the CTA's work ends from the chunk records.
  const int n_units_all = n_items * Hkv;
  const int per_cta_w = (n_units_all + (int)gridDim.x - 1) / (int)gridDim.x;  // whole units per CTA
  const bool fast = !UMMA && MT == 1 && p.whole_units && p.n_qt == 1 && (per_cta_w + Hkv - 1) / Hkv + 1 <= 32;
  if (fast) {
    fence_proxy_async();  // generic-proxy zero fill before async-proxy (TMA) writes to the same bytes
    __syncthreads();      // barriers initialised, V slots zeroed: nothing here depends on an earlier kernel
  }
  // Early K/V (whole-unit decode, p.early_kv): the host knows that nothing of the pool this launch
  // reads - lengths, block table, pages - was written by the kernel in front of it on the stream.
  // The two warps that issue copies then skip the wait here: they look the unit up and send its
  // first K/V chunks while the kernel in front is still in its tail, and wait only before the
  // first thing that does depend on that kernel (the query rows, the pending rows, a write to out).
  // gdc_open: this thread has not waited for the kernel in front yet.
  bool gdc_open = fast && p.early_kv && warp >= NW;
  auto gdc_wait = [&]() {
    if (gdc_open) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
      gdc_open = false;
    }
  };
  if (!gdc_open) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // A kernel launched as a programmatic dependent of this one (the next layer's attention launch, or
    // its K/V append, which touches nothing this kernel reads or writes) may start once every CTA is
    // past this point.  The trigger comes after the wait on purpose: a dependent that starts then knows
    // that the kernel in front of this one has completed, which is what keeps two launches that use the
    // workspace apart (see the appends' trailing wait) and what lets a dependent trust everything older.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }
  const int cta = blockIdx.x;
  long long T = 0, x0 = 0, x1 = 0;
  int NC = 1, n_my = 0;
  bool small = true;
  // range boundaries floor(T * c / NC); 32-bit arithmetic whenever it cannot overflow
  auto range_begin = [&](int c) -> long long {
    return small ? (long long)((unsigned)T * (unsigned)c / (unsigned)NC) : T * c / NC;
  };
  auto cta_of = [&](long long x) -> int {  // the CTA whose range holds chunk x
    return small ? (int)(((unsigned)(x + 1) * (unsigned)NC + (unsigned)T - 1u) / (unsigned)T) - 1
                 : (int)(((x + 1) * NC + T - 1) / T) - 1;
  };
  PageWindow pw;
  int pw_slot = -1;  // short prologue: the sequence whose first block-table window is already loaded
  int fast_it0 = 0, fast_it1 = -1;
  int n_spec = 0;  // short prologue: ring stages whose copies went out before the length was known
  const uint32_t page_box_bytes = (uint32_t)p.box_rows * 128u * 2u * HALVES;  // K and V boxes of one page
  int q_spec = 0;  // ... and whether the unit's query rows went out with them
  if (fast) {
    const int u0 = cta * per_cta_w, u1 = min(n_units_all, u0 + per_cta_w);
    if (u0 >= n_units_all) return;  // (known from the CTA index: every thread leaves)
    n_my = INT_MAX;                 // consumers run until the record of the CTA's last chunk
    // A CTA with a single unit of one-page chunks: the copies of the unit's first pages and of its query
    // rows leave before its length is known - a first page that is in the table holds keys unless the
    // sequence is empty, and pages that turn out to lie beyond the length are received and dropped by
    // the producer.  The epilogue warp, idle until the first unit is done, issues them while the
    // producer warp works out the unit's chunks: one warp's couple of microseconds of dependent scalar
    // work then runs beside the DRAM latency of the first copies, not in front of it.
    const bool spec_ok = u1 - u0 == 1 && p.pages_per_chunk == 1 && p.kv.block_table && !p.q_lens;
    if (warp == NW + 1 && spec_ok) {
      const int b0 = u0 / Hkv, h0s = u0 - b0 * Hkv;
      const int slot0 = view_slot(p.kv, b0);
      const int want = min(n_stages, 4);
      int n = 0, qs = 0;
      if (slot0 >= 0) {
        int pg = -1;
        if (lane < want && lane < p.kv.max_pages_per_seq) {
          pg = __ldcg(p.kv.block_table + (size_t)slot0 * p.kv.max_pages_per_seq + lane);
          if (pg >= p.kv.n_pages) pg = -1;
        }
        const unsigned have = __ballot_sync(0xffffffffu, pg >= 0);
        n = __ffs(~have) - 1;  // leading pages that are in the table
        if (pend) {
          // (the page that takes the pending row is copied only after the row has been stored: lane 31
          // fetches the length beside the other lanes' table entries)
          int len0 = lane == 31 ? view_len(p.kv, slot0) : 0;
          len0 = __shfl_sync(0xffffffffu, len0, 31);
          n = min(n, len0 / P);
        }
        const int is_v = lane & 1, hf = (lane >> 1) % HALVES;
        for (int c = 0; c < n; ++c) {
          const int pgc = __shfl_sync(0xffffffffu, pg, c);
          if (lane < 2 * HALVES)
            tma_load_4d_hint(ring + (size_t)c * STAGE + (is_v ? KVB : 0) + hf * HALF_B, is_v ? &tmV : &tmK, hf * 64, 0,
                             pgc * Hkv + h0s, is_v ? p.c3_v : p.c3_k, &full_bar[c], l2_evict_first_policy());
        }
        qs = n > 0;
      }
      if (lane == 0) {
        misc[3] = n;
        misc[7] = qs;
      }
      __syncwarp();
      asm volatile("bar.arrive 2, 64;" ::: "memory");  // the producer picks the two numbers up behind this
      if (gdc_open) {
        // Early K/V: the query rows (and the pending rows) may still be on their way from the kernel in
        // front, so they are not READ before the wait below - but asking L2 for their lines is harmless
        // whatever that kernel does to them afterwards (L2 is where its writes land), and when they have
        // been sitting in DRAM it takes a DRAM round trip off the path from that kernel's end to this
        // launch's first chunk.
        const int q_rows = min(MR, p.q_len * G);
        const int r = lane >> 1, sq = r / G, g = r - sq * G;  // two 128-byte lines per row of 128 elements
        if (r < q_rows && (lane & 1) * 64 < D)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(p.q + (size_t)b0 * p.q_sb + (size_t)(h0s * G + g) * p.q_sh +
                                                        (size_t)sq * p.q_ss + (lane & 1) * 64));
        if (pend && lane >= 28 && (lane & 1) * 64 < D)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(((lane & 2) ? p.v_pend : p.k_pend) + (size_t)b0 * p.pend_sb +
                                                        (size_t)h0s * p.pend_sh + (lane & 1) * 64));
      }
      gdc_wait();  // (early K/V: the page copies above are out; what follows reads the step's own inputs)
      if (qs) {
        const int q_rows = min(MR, p.q_len * G);
        for (int r = lane; r < q_rows; r += 32) {
          const int sq = r / G, g = r - sq * G;
          bulk_g2s(qbuf + r * QS, p.q + (size_t)b0 * p.q_sb + (size_t)(h0s * G + g) * p.q_sh + (size_t)sq * p.q_ss,
                   D * 2u, &full_bar[0]);
        }
      }
    }
    if (warp == NW + 1) {
      gdc_wait();
      if (pend) {
        // the pending rows of this CTA's units go into the pool now, long before the producer reaches
        // the chunks that hold them; it picks the all-clear up at named barrier 4
        bool ok_rows = true;
        for (int u = u0; u < u1; ++u) ok_rows &= store_pending_row<D>(p, u / Hkv, u - (u / Hkv) * Hkv, lane);
        if (!ok_rows && lane == 0) raise_status(p.kv.status, PACE_DEV_BAD_INDEX);
        fence_proxy_async_all();
        __syncwarp();
        asm volatile("bar.arrive 4, 64;" ::: "memory");
      }
    }
    if (warp == NW) {
      const int it0 = u0 / Hkv, it1 = (u1 - 1) / Hkv;
      fast_it0 = it0;
      fast_it1 = it1;
      const int b = it0 + lane;  // one lane per sequence this CTA touches
      int n = 0, slot = -1, len = 0;
      // (the pool's status word travels beside the lengths: where an earlier launch ran out of patience,
      // this one streams nothing and writes nothing until the host has cleared the word)
      const int status_word = lane == 31 ? load_status_word(p.kv.status) : 0;
      if (b <= it1) {
        slot = view_slot(p.kv, b);
        if (slot >= 0) len = view_len(p.kv, slot) + (pend ? 1 : 0);
      }
      // the first sequence's block-table window: its loads go out right behind the loads of the
      // lengths, before anything waits for either
      const int slot0 = __shfl_sync(0xffffffffu, slot, 0);
      if (slot0 >= 0) {
        const int step0 = p.pages_per_chunk > 0 ? (32 / p.pages_per_chunk) * p.pages_per_chunk : 32;
        pw.start(p.kv, slot0, 0, step0, lane);
        pw_slot = slot0;
      }
      if (b <= it1) {
        const int S = p.q_lens ? min(p.q_lens[b], p.q_len) : p.q_len;
        sb_slot[b] = slot;
        sb_len[b] = len;
        sb_kvs[b] = p.kv_start ? p.kv_start[b] : 0;
        sb_S[b] = S;
        if (slot >= 0 && S > 0) {
          const int s_hi = min(S - 1, (MR - 1) / G);
          const int hi = p.causal ? len - S + s_hi + 1 : len;
          n = chunks_of_m(p, min(hi, len)) * Hkv;
        }
      }
      int v = n;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
      }
      // chunk coordinates local to this CTA: the first sequence it touches starts at 0
      if (b <= it1) prefix[b + 1] = v;
      if (lane == 0) prefix[it0] = 0;
      __syncwarp();
      const int h0 = u0 - it0 * Hkv, h1 = (u1 - 1) - it1 * Hkv;
      x0 = (long long)prefix[it0] + (long long)h0 * ((prefix[it0 + 1] - prefix[it0]) / Hkv);
      x1 = (long long)prefix[it1] + (long long)(h1 + 1) * ((prefix[it1 + 1] - prefix[it1]) / Hkv);
      const bool gave_up = pool_gave_up(__shfl_sync(0xffffffffu, status_word, 31));
      // query rows that see no key at all (nothing cached) get zeros
      for (int u = u0; u < u1 && !gave_up; ++u) {
        const int it = u / Hkv, h = u - it * Hkv;
        if (prefix[it + 1] != prefix[it]) continue;
        gdc_wait();  // (early K/V: a write to out)
        const int R = sb_S[it] * G;
        for (int o = lane; o < MR * D; o += 32) {
          const int r = o / D, d = o % D;
          if (r < R) {
            const int sq = r / G, g = r - sq * G;
            p.out[(size_t)it * p.o_sb + (size_t)(h * G + g) * p.o_sh + (size_t)sq * p.o_ss + d] = __float2bfloat16(0.f);
          }
        }
      }
      n_my = gave_up ? 0 : (int)(x1 - x0);
      if (gave_up && lane == 0) *abort = 1;
      if (spec_ok) {
        asm volatile("bar.sync 2, 64;" ::: "memory");
        n_spec = misc[3];
        q_spec = misc[7];
      }
      if (n_my <= 0) {
        // nothing to stream: a record that says so for the consumers, a result slot that says so for
        // the epilogue warp
        if (lane == 0) {
          metas[0].flags = 8;
          if (n_spec > 0) {  // (the record travels with the first speculative copy; the others are received here)
            for (int k = 0; k < n_spec; ++k)
              mbar_arrive_expect_tx(&full_bar[k],
                                    page_box_bytes + ((k == 0 && q_spec) ? (uint32_t)min(MR, p.q_len * G) * D * 2u : 0u));
            for (int k = 0; k < n_spec; ++k) mbar_wait(&full_bar[k], 0);
          } else {
            mbar_arrive(&full_bar[0]);
          }
          float* rden0 = reinterpret_cast<float*>(res) + p.live_max * D + p.live_max;
          reinterpret_cast<ResMeta*>(rden0 + p.live_max)->last_part = 1;
          for (int k = 0; k < NW; ++k) mbar_arrive(&res_full[0]);
        }
        return;
      }
    }
  } else {
  // ---- prologue, part 2: per-sequence lengths -> chunk prefix -> this CTA's range ----
  const int status_word = tid == NTHR - 1 ? load_status_word(p.kv.status) : 0;  // (looked at behind the loads below)
  int my_slot[(kMaxItems + NTHR - 1) / NTHR];
  int my_len[(kMaxItems + NTHR - 1) / NTHR];
#pragma unroll
  for (int r = 0; r < (kMaxItems + NTHR - 1) / NTHR; ++r) {
    const int b = tid + r * NTHR;
    my_slot[r] = -1;
    my_len[r] = 0;
    if (b < p.batch) {
      my_slot[r] = view_slot(p.kv, b);
      if (my_slot[r] >= 0) {
        my_len[r] = view_len(p.kv, my_slot[r]) + (pend ? 1 : 0);
        // the producer will walk this row of the block table a few microseconds from now: start
        // bringing its first lines into L2 (the K/V stream of the previous launch has evicted them)
        if (p.kv.block_table) {
          const char* row = reinterpret_cast<const char*>(p.kv.block_table + (size_t)my_slot[r] * p.kv.max_pages_per_seq);
          const int bytes = min(p.kv.max_pages_per_seq * 4, 512);
          for (int o = 0; o < bytes; o += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(row + o));
        }
      }
      sb_kvs[b] = p.kv_start ? p.kv_start[b] : 0;
      sb_S[b] = p.q_lens ? min(p.q_lens[b], p.q_len) : p.q_len;
    }
  }
#pragma unroll
  for (int r = 0; r < (kMaxItems + NTHR - 1) / NTHR; ++r) {
    const int b = tid + r * NTHR;
    if (b < p.batch) {
      sb_slot[b] = my_slot[r];
      sb_len[b] = my_len[r];
    }
  }
  fence_proxy_async();  // generic-proxy zero fill before async-proxy (TMA) writes to the same bytes
  // an earlier launch on this pool ran out of patience: nothing is attempted until the host clears that
  if (__syncthreads_or(pool_gave_up(status_word))) return;
  int saw_empty = 0;
  for (int it = tid; it < n_items; it += NTHR) {
    const int b = p.n_qt == 1 ? it : it / p.n_qt, qt = it - b * p.n_qt;
    int n = 0;
    if (sb_slot[b] >= 0) {
      const int S = sb_S[b], R = S * G;
      if (qt * MR < R) {
        const int kv_len = sb_len[b];
        const int s_hi = min(S - 1, ((qt + 1) * MR - 1) / G);
        const int hi = p.causal ? kv_len - S + s_hi + 1 : kv_len;
        n = chunks_of_m(p, min(hi, kv_len)) * Hkv;
      }
    }
    prefix[it + 1] = n;
    saw_empty |= (n == 0);
    if (n > 0) atomicMax(&misc[2], n / Hkv);
  }
  const int any_empty = __syncthreads_or(saw_empty);
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < n_items; base += 32) {
      const int i = base + lane;
      int v = i < n_items ? prefix[i + 1] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
      }
      if (i < n_items) prefix[i + 1] = v + carry;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
    if (lane == 0) prefix[0] = 0;
  }
  __syncthreads();
  T = prefix[n_items];
  NC = (long long)gridDim.x < T ? (int)gridDim.x : (int)T;
  small = (T + 1) * (NC + 1) < (1LL << 31);
  x0 = cta < NC ? range_begin(cta) : 0;
  x1 = cta < NC ? range_begin(cta + 1) : 0;
  // When giving every CTA the same number of WHOLE units keeps the busiest CTA within 1.3x of an equal share of the
  // chunks, do that instead: a little more streaming for the busiest CTA (and some SMs idle), but no unit
  // is cut, so nothing is published to and merged from the workspace and no CTA waits for a last
  // arriver.  (Batch 32 x 8 KV heads: on 148 eight-warp CTAs, two units each, measured 22.5 us against
  // 23.5 us for the chunk-balanced partition; on 296 four-warp CTAs, one unit each and 1.24x the equal
  // share, 19.1 us against 19.6 us.  PARD verify, 128 units: 24.9 us against 34.0 us.)
  const int n_units = n_items * Hkv;
  const int per_cta = (n_units + (int)gridDim.x - 1) / (int)gridDim.x;  // whole units per CTA
  // p.whole_units: the caller asked for this form whatever the balance; such a launch never touches
  // the workspace.
  if (p.whole_units || (long long)per_cta * misc[2] * gridDim.x * 10 <= T * 13) {
    x0 = x1 = 0;
    const int u0 = cta * per_cta, u1 = min(n_units, u0 + per_cta);
    if (u0 < n_units) {
      const int it0 = u0 / Hkv, h0 = u0 - it0 * Hkv;
      x0 = (long long)prefix[it0] + (long long)h0 * ((prefix[it0 + 1] - prefix[it0]) / Hkv);
      const int it1 = (u1 - 1) / Hkv, h1 = (u1 - 1) - it1 * Hkv;
      x1 = (long long)prefix[it1] + (long long)(h1 + 1) * ((prefix[it1 + 1] - prefix[it1]) / Hkv);
    }
  }

  // query rows that see no key at all (nothing cached) get zeros
  for (int u = cta; any_empty && u < n_items * Hkv; u += gridDim.x) {
    const int it = u / Hkv, h = u - it * Hkv;
    if (prefix[it + 1] != prefix[it]) continue;
    const int b = it / p.n_qt, qt = it - b * p.n_qt;
    const int R = sb_S[b] * G;
    for (int o = tid; o < MR * D; o += NTHR) {
      const int r = qt * MR + o / D, d = o % D;
      if (r < R) {
        const int s = r / G, g = r - s * G;
        p.out[(size_t)b * p.o_sb + (size_t)(h * G + g) * p.o_sh + (size_t)s * p.o_ss + d] = __float2bfloat16(0.f);
      }
    }
  }
  if (x1 <= x0) return;
  n_my = (int)(x1 - x0);
  }  // general prologue

  if (warp == NW) {
    // ================================ producer ================================
    // One warp feeds the ring.  Everything costly (table walks, divisions, the partition
    // arithmetic, the 48-byte part record) happens once per unit part; one iteration of the
    // chunk loop is a few dozen instructions, because a single warp's dependent instruction
    // stream is what paces the whole pipeline.
    // the item holding chunk x0: the last one whose prefix is <= x0; 32 candidates per ballot
    int it = 0;
    if (fast) {
      const int k = fast_it0 + lane;
      const unsigned m = __ballot_sync(0xffffffffu, k <= fast_it1 && (long long)prefix[k] <= x0);
      it = fast_it0 + 31 - __clz(m);  // (lane 0 always votes: prefix[it0] = 0)
    } else
    for (int base = 0; base < n_items; base += 32) {
      const int k = base + lane;
      const unsigned m = __ballot_sync(0xffffffffu, k < n_items && (long long)prefix[k] <= x0);
      if (m == 0) break;
      it = base + 31 - __clz(m);
      if (m != 0xffffffffu) break;
    }
    int nch = (prefix[it + 1] - prefix[it]) / Hkv;
    const int rel = (int)(x0 - prefix[it]);
    int h = rel / nch;
    int j = rel - h * nch;
    const bool whole_pages = p.pages_per_chunk > 0;
    const int is_v = lane & 1;
    const int hf = (lane >> 1) % HALVES;
    const int pi = whole_pages ? lane / (2 * HALVES) : 0;
    const bool copier = whole_pages ? (lane < 2 * HALVES * p.pages_per_chunk) : (lane < 2 * HALVES);
    const CUtensorMap* tm = is_v ? &tmV : &tmK;
    const int c3 = is_v ? p.c3_v : p.c3_k;
    const int c0 = hf * 64;
    const uint32_t lane_off =
        UMMA ? (is_v ? (uint32_t)n_stages * KVB + hf * HALF_B : (uint32_t)hf * n_stages * HALF_B) + (uint32_t)pi * P * 128
             : (uint32_t)(is_v ? KVB : 0) + hf * HALF_B + (uint32_t)pi * P * 128;
    const uint32_t stage_step = UMMA ? (is_v ? KVB : HALF_B) : STAGE;  // bytes from one stage's tile to the next
    const int win_step = whole_pages ? (32 / p.pages_per_chunk) * p.pages_per_chunk : 32;
    const uint32_t box_bytes = page_box_bytes;
    const uint64_t stream_policy = l2_evict_first_policy();
    const int CT = p.chunk_tokens;
    int i = 0, s = 0, ph = 0, part_idx = 0;
    bool ok = true;
    // Early K/V: the query rows of the first unit part are the first thing this warp touches that the
    // kernel in front may have written.  Their copies are held back - the part's K/V chunks go out
    // first - until the warp would block anyway, then it waits for that kernel and sends them.
    // dq_*: the copies held back.
    int dq_b = -1, dq_h = 0, dq_r_lo = 0, dq_rows = 0, dq_s = 0;
    auto send_q_rows = [&](int b, int h, int r_lo, int q_rows, uint64_t* bar) {
      for (int r = lane; r < q_rows; r += 32) {
        const int rr = r_lo + r, sq = rr / G, g = rr - sq * G;
        const __nv_bfloat16* src = p.q + (size_t)b * p.q_sb + (size_t)(h * G + g) * p.q_sh + (size_t)sq * p.q_ss;
        bulk_g2s(qbuf + r * QS, src, D * 2u, bar);
      }
    };
    auto flush_q = [&]() {
      gdc_wait();
      if (dq_b >= 0) send_q_rows(dq_b, dq_h, dq_r_lo, dq_rows, &full_bar[dq_s]);
      dq_b = -1;
    };
    bool rows_stored = false;  // short prologue with a pending row: the epilogue warp's all-clear has been picked up
    while (i < n_my && ok) {
      const int b = p.n_qt == 1 ? it : it / p.n_qt, qt = it - b * p.n_qt;
      const int slot = sb_slot[b];
      const int kv_len = sb_len[b];
      const int S = sb_S[b];
      const int R = S * G;
      const int r_lo = qt * MR;
      const int s_hi = min(S - 1, (r_lo + MR - 1) / G);
      const int len = min(kv_len, p.causal ? kv_len - S + s_hi + 1 : kv_len);  // keys this tile can see
      const int j_end = min(nch, j + (n_my - i));
      int lp, row0;  // the chunk's first logical page (uniform) and first row inside it
      if (whole_pages) {
        lp = j * p.pages_per_chunk;
        row0 = 0;
      } else {
        lp = j / p.chunks_per_page;
        row0 = (j - lp * p.chunks_per_page) * kChunk;
      }
      const bool loaded = pw_slot == slot && lp == 0;  // (short prologue: the first window may be here already)
      pw_slot = -1;
      if (!loaded) pw.start(p.kv, slot, lp, win_step, lane);  // loads in flight while the arithmetic below runs
      int mode = 0, parts = 1, first_cta = cta, first_slot = 0;
      {
        const long long ub = (long long)prefix[it] + (long long)h * nch, ue = ub + nch;
        if (ub < x0 || ue > x1) {
          first_cta = ub >= x0 ? cta : cta_of(ub);
          const int last_cta = ue <= x1 ? cta : cta_of(ue - 1);
          parts = last_cta - first_cta + 1;
          first_slot = (ub >= x0 ? x0 : range_begin(first_cta)) == ub ? 0 : 1;
          mode = (cta == first_cta) ? (first_slot ? 2 : 1) : 1;
        }
      }
      const int q_rows = min(MR, R - r_lo);
      const int c2h = h;
      if (!UMMA && part_idx > 0) {
        flush_q();
        if (!mbar_wait(q_empty, (part_idx - 1) & 1, abort)) { ok = false; break; }
      }
      for (bool first = true; j < j_end; ++j, ++i, first = false) {
        if (i >= n_stages) {
          if (!UMMA && MT == 1) flush_q();
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort)) { ok = false; break; }
        }
        const int tok0 = whole_pages ? j * CT : lp * P + row0;
        const int rows = whole_pages ? min(CT, len - tok0) : min(min(kChunk, P - row0), len - tok0);
        const int n_pages_c = !whole_pages ? 1 : (rows == CT ? p.pages_per_chunk : (rows + P - 1) / P);
        const bool last = (j == j_end - 1);
        // A partly filled page of 64 tokens (a sequence's last one) is fetched in boxes of 16 rows, one
        // lane each, through a second tensor map: a whole-page box would bring up to 63 rows from DRAM
        // that nobody reads (one launch of batch 32 at 515 cached tokens reads 13 % more than it needs).
        // Rows of the stage that no box covers keep what an earlier chunk left there: finite numbers,
        // masked out of the scores and multiplied by zero weights.
        const bool sub = !UMMA && MT == 1 && p.sub_boxes && rows <= kChunk - 16 && i >= n_spec;
        const int n_sub = (rows + 15) >> 4;
        if (lane == 0) {
          MetaM* m = &metas[s];
          *reinterpret_cast<int4*>(m) = make_int4(
              rows, tok0, (first ? 1 : 0) | (last ? 2 : 0) | ((last && i == n_my - 1) ? 4 : 0), sb_kvs[b]);
          if (first) {
            *reinterpret_cast<int4*>(&m->b) = make_int4(b, h, r_lo, R);
            *reinterpret_cast<int4*>(&m->kv_len) = make_int4(kv_len, S, mode, parts);
            *reinterpret_cast<int4*>(&m->first_cta) = make_int4(first_cta, first_slot, it * Hkv + h, j_end - j);
          }
          mbar_arrive_expect_tx(&full_bar[s], (sub ? (uint32_t)n_sub * (box_bytes / 4u) : (uint32_t)n_pages_c * box_bytes) +
                                                  ((first && !UMMA) ? (uint32_t)q_rows * D * 2u : 0u));
        }
        __syncwarp();
        const int pg = pw.get(sub ? lp : lp + pi, lp, lane);
        if (pend && j == nch - 1) {
          // The unit's final chunk holds the pending row, which has to be in the pool before the copy
          // leaves.  Short prologue: the epilogue warp stored this CTA's rows at the start (one
          // meeting, once).  General prologue: this warp stores the unit's row itself, now.
          if (fast) {
            if (!rows_stored) asm volatile("bar.sync 4, 64;" ::: "memory");
            rows_stored = true;
          } else {
            if (!store_pending_row<D>(p, b, h, lane) && lane == 0) raise_status(p.kv.status, PACE_DEV_BAD_INDEX);
            fence_proxy_async_all();
            __syncwarp();
          }
        }
        if (i < n_spec) {
          // (short prologue: this chunk's copy is on its way already - same sequence, head and page)
        } else if (sub) {
          // lane = (16-row box, K | V, column block): the same lane order as for pages of a chunk
          const int bx = lane / (2 * HALVES);
          if (bx < n_sub) {
            if (pg >= 0)
              tma_load_4d_hint(ring + (size_t)s * STAGE + (is_v ? KVB : 0) + hf * HALF_B + bx * 16 * 128, &tmS, c0, bx * 16,
                               pg * Hkv + c2h, c3, &full_bar[s], stream_policy);
            else raise_status(p.kv.status, PACE_DEV_BAD_INDEX);
          }
        } else if (copier && pi < n_pages_c) {
          if (pg >= 0) {
            if (p.n_qt == 1) tma_load_4d_hint(ring + (size_t)s * stage_step + lane_off, tm, c0, row0, pg * Hkv + c2h, c3, &full_bar[s], stream_policy);
            else tma_load_4d(ring + (size_t)s * stage_step + lane_off, tm, c0, row0, pg * Hkv + c2h, c3, &full_bar[s]);
          }
          else raise_status(p.kv.status, PACE_DEV_BAD_INDEX);  // the consumers' bounded wait on this stage gives up
        }
        if (first && !UMMA && !(q_spec && i == 0)) {  // (the tcgen05 variant's softmax warps write the Q tile themselves, swizzled)
          if (gdc_open) {
            dq_b = b, dq_h = h, dq_r_lo = r_lo, dq_rows = q_rows, dq_s = s;
          } else {
            send_q_rows(b, h, r_lo, q_rows, &full_bar[s]);
          }
        }
        if (whole_pages) {
          lp += p.pages_per_chunk;
        } else {
          row0 += kChunk;
          if (row0 >= P) { row0 = 0; ++lp; }
        }
        if (++s == n_stages) { s = 0; ph ^= 1; }
      }
      if (!ok) break;
      if (!UMMA && MT == 1) flush_q();
      ++part_idx;
      j = 0;
      if (i >= n_my) break;
      if (++h == Hkv) {
        h = 0;
        ++it;
        while (it < n_items && prefix[it + 1] == prefix[it]) ++it;
        if (it >= n_items) break;
        nch = (prefix[it + 1] - prefix[it]) / Hkv;
      }
    }
    if (!ok && lane == 0) {
      raise_status(p.kv.status, PACE_DEV_WAIT_TIMEOUT);
      // let copies already in flight land before the CTA's shared memory is released
      const int from = i > n_stages ? i - n_stages : 0;
      for (int k = from; k < i; ++k) mbar_wait(&full_bar[k % n_stages], (k / n_stages) & 1);  // (never cut short)
    }
    if (lane == 0 && i < n_spec) {
      // speculative copies of pages beyond the unit's length: nobody consumes them, receive them here
      for (int k = i; k < n_spec; ++k) mbar_arrive_expect_tx(&full_bar[k], page_box_bytes);
      for (int k = i; k < n_spec; ++k) mbar_wait(&full_bar[k], 0);
    }
    return;
  }

  if constexpr (UMMA) {
    // ========= tcgen05 variant: softmax warps 0..7 (two groups), MMA issuer warps 9 (QK) and 10 (PV) =========
    UmmaCtx uc;
    uc.ring = ring;
    uc.metas = metas;
    uc.full_bar = full_bar;
    uc.empty_bar = empty_bar;
    uc.s_full = umma_bars;
    uc.p_full = umma_bars + 4;
    uc.s_free = umma_bars + 6;
    uc.o_full = umma_bars + 8;
    uc.q_ready = umma_bars + 10;
    uc.drain = umma_bars + 11;
    uc.pub = umma_bars + 13;
    uc.xch = umma_bars + 14;
    uc.drain_b = umma_bars + 15;
    uc.tmem_slot = reinterpret_cast<uint32_t*>(misc + 5);
    uc.flag = misc + 6;
    uc.abort = misc + 4;
    uc.n_my = n_my;
    uc.n_stages = n_stages;
    uc.cta = cta;
    uc.qsw = qbuf;
    umma_consumer<D, WIDE>(p, uc, tid);
    return;
  }

  if (warp == NW + 1) {
    // ================================ epilogue warp ================================
    // Takes each finished unit part from shared memory to global memory: the output rows, or an
    // fp32 partial plus the arrival count (and the merge, when this CTA arrives last).  The global
    // round trips happen here, off the consumers' path.
    for (int k = 0;; ++k) {
      const int rs = k % sp.n_res;
      if (!mbar_wait(&res_full[rs], (k / sp.n_res) & 1, abort)) {
        if (lane == 0) raise_status(p.kv.status, PACE_DEV_WAIT_TIMEOUT);
        return;
      }
      const float* rnum = reinterpret_cast<const float*>(res + (size_t)rs * sp.res_slot_bytes);
      const float* rM = rnum + p.live_max * D;
      const float* rden = rM + p.live_max;
      const ResMeta rm = *reinterpret_cast<const ResMeta*>(rden + p.live_max);
      if (rm.last_part) break;  // the CTA's last part is published by the consumer warps themselves
      publish_part<D, MR, 32, true>(p, rm, rnum, rM, rden, lane, cta, nullptr);
      __syncwarp();
      if (lane == 0) mbar_arrive(&res_empty[rs]);
    }
    return;
  }

  // ================================= consumers =================================
  const int mt = warp / NS, ns = warp - mt * NS;
  const int qr = lane >> 2, qc = lane & 3;  // fragment row within 8, column pair
  uint32_t qa[KS][4];
  float o[ON][4];
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  int lim0 = INT_MAX, lim1 = INT_MAX;  // first key NOT visible to my two rows
  int srow0 = 0, srow1 = 0, bcur = 0;  // query token of my two rows (additive-mask lookup)
  int n_parts_done = 0;
  // Decode tiles of at most 8 live rows (grouped heads x tokens) are computed transposed: S^T = K Q^T and
  // O^T = V^T P^T, keys and head dimensions on the 16-row side of m16n8k16 and the query rows on its 8-column
  // side.  Half the MMAs of the 16-row tile for the same keys (mma.sync runs at one m16n8k16 per 16 cycles
  // and scheduler here, and the consumers' chunk time is mostly those), half the accumulator registers.
  // Same variables, other meaning: qa[k][0..1] is the B fragment of Q^T, o[t] the tile of 16 head
  // dimensions x 8 query rows, m0/l0 and m1/l1 belong to query rows 2 * qc and 2 * qc + 1.
  bool tr = false;
  ResMeta fin;  // the current unit part, read from the part record of its first chunk
  fin.last_part = 0;
#pragma unroll
  for (int n = 0; n < ON; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
#pragma unroll
  for (int k = 0; k < KS; ++k) qa[k][0] = qa[k][1] = qa[k][2] = qa[k][3] = 0u;

  for (int i = 0; i < n_my; ++i) {
    const int s = i % n_stages;
    if (!mbar_wait(&full_bar[s], (i / n_stages) & 1, abort)) {
      if (lane == 0) raise_status(p.kv.status, PACE_DEV_WAIT_TIMEOUT);
      return;
    }
    const unsigned char* st = ring + (size_t)s * STAGE;
    const MetaM* meta = &metas[s];
    const int rows = meta->rows, tok0 = meta->tok0, flags = meta->flags, kvs = meta->kvs;
    if (flags & 8) return;  // (short prologue: the producer found nothing to stream)

    if (flags & 1) {
      // ---- new unit part: Q fragments to registers, per-row visibility limits ----
      const int R = meta->R, r_lo = meta->r_lo, kv_len = meta->kv_len, S = meta->S;
      tr = MT == 1 && 1 && R - r_lo <= 8 && !p.mask;
      const uint32_t qb = smem_u32(qbuf) + (uint32_t)(mt * 16) * QS;
      if (tr) {
        // B fragments of Q^T (16 head dimensions x 8 query rows): thread holds row qr, dimensions 2 qc + {0, 1} (+ 8)
        const unsigned char* qrow = qbuf + qr * QS + qc * 4;
#pragma unroll
        for (int k = 0; k < KS; ++k) {
          qa[k][0] = *reinterpret_cast<const uint32_t*>(qrow + k * 32);
          qa[k][1] = *reinterpret_cast<const uint32_t*>(qrow + k * 32 + 16);
        }
      } else {
#pragma unroll
        for (int k = 0; k < KS; ++k) {
          const int mi = lane >> 3;
          const int row = (mi & 1) * 8 + (lane & 7);
          const int cch = k * 2 + (mi >> 1);
          ldsm_x4(qb + row * QS + cch * 16, qa[k][0], qa[k][1], qa[k][2], qa[k][3]);
        }
      }
      m0 = m1 = -INFINITY;
      l0 = l1 = 0.f;
#pragma unroll
      for (int n = 0; n < ON; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
      __syncwarp();
      if (lane == 0) mbar_arrive(q_empty);
      // (transposed: my two query rows are 2 qc and 2 qc + 1, the columns of my accumulators)
      const int r0 = tr ? r_lo + 2 * qc : r_lo + mt * 16 + qr, r1 = tr ? r0 + 1 : r0 + 8;
      srow0 = r0 / G;
      srow1 = r1 / G;
      lim0 = (r0 < R) ? (p.causal ? kv_len - S + srow0 + 1 : kv_len) : INT_MAX;
      lim1 = (r1 < R) ? (p.causal ? kv_len - S + srow1 + 1 : kv_len) : INT_MAX;
      bcur = meta->b;
      fin.b = meta->b;
      fin.h = meta->h;
      fin.r_lo = r_lo;
      fin.live = min(MR, R - r_lo);
      fin.mode = meta->mode;
      fin.parts = meta->parts;
      fin.first_cta = meta->first_cta;
      fin.first_slot = meta->first_slot;
      fin.unit = meta->unit;
    }

    // The chunk's keys are dealt to the NS warps of a row tile in equal slices of whole 8-key tiles:
    // a short chunk (a page of 33..63 tokens, a sequence's last chunk) keeps every warp busy instead of
    // filling the first slices only.  Row tiles made of padding rows only sit the chunk out.
    int tw = TW;
    if (SL > 1 && NT > 1 && rows < kChunk) tw = min(TW, (((rows + SL - 1) / SL) + 7) & ~7);
    const int tw0 = (ns % SL) * tw;
    const bool mine = (i % DG) == (ns / SL);
    if (mine && tw0 < rows && mt * 16 < fin.live) {
      const uint32_t kb = smem_u32(st), vb = kb + KVB;
      if (tr) {
        // ---- S^T = K Q^T: my 16 keys x 8 query rows, two accumulators over the k-steps ----
        const int mi = lane >> 3;
        float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
        {
          const int row = tw0 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
          for (int k = 0; k < KS; ++k) {
            const int cg = k * 2 + (mi >> 1);
            uint32_t a[4];
            ldsm_x4(kb + (cg >> 3) * HALF_B + row * 128 + (((cg & 7) ^ (row & 7)) << 4), a[0], a[1], a[2], a[3]);
            mma16816((k & 1) ? sb : sa, a, qa[k][0], qa[k][1]);
          }
        }
        // sc[0], sc[1]: key qr, query rows 2 qc and 2 qc + 1; sc[2], sc[3]: key qr + 8
        float sc[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[e] = (sa[e] + sb[e]) * p.scale_log2;
        {
          // keys outside my slice of the chunk, outside the chunk, left padding, beyond the row's limit
          const int kk0 = tw0 + qr, kk1 = kk0 + 8;
          const int t0 = tok0 + kk0, t1 = tok0 + kk1;
          const bool in0 = qr < tw && kk0 < rows && t0 >= kvs, in1 = qr + 8 < tw && kk1 < rows && t1 >= kvs;
          if (!(in0 && t0 < lim0)) sc[0] = -INFINITY;
          if (!(in0 && t0 < lim1)) sc[1] = -INFINITY;
          if (!(in1 && t1 < lim0)) sc[2] = -INFINITY;
          if (!(in1 && t1 < lim1)) sc[3] = -INFINITY;
        }
        // ---- online softmax down the key side: my two keys, then the 8 lanes that share my query rows ----
        float mx0 = fmaxf(sc[0], sc[2]), mx1 = fmaxf(sc[1], sc[3]);
#pragma unroll
        for (int o_ = 4; o_ < 32; o_ <<= 1) {
          mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o_));
          mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o_));
        }
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float a0 = (m0 == -INFINITY) ? 0.f : fast_exp2(m0 - n0);
        const float a1 = (m1 == -INFINITY) ? 0.f : fast_exp2(m1 - n1);
        const float e0 = (n0 == -INFINITY) ? 0.f : n0, e1 = (n1 == -INFINITY) ? 0.f : n1;
        m0 = n0;
        m1 = n1;
        const float p00 = fast_exp2(sc[0] - e0), p01 = fast_exp2(sc[1] - e1);
        const float p10 = fast_exp2(sc[2] - e0), p11 = fast_exp2(sc[3] - e1);
        l0 = l0 * a0 + p00 + p10;  // (this thread's keys only: summed over the lanes at the end of the part)
        l1 = l1 * a1 + p01 + p11;
#pragma unroll
        for (int t = 0; t < D / 16; ++t) {
          o[t][0] *= a0;
          o[t][1] *= a1;
          o[t][2] *= a0;
          o[t][3] *= a1;
        }
        // P (keys x query rows) -> B fragments of P^T: one 8x8 transpose per 8 keys
        const uint32_t pb0 = movmatrix_t(f2_to_bf2(p00, p01)), pb1 = movmatrix_t(f2_to_bf2(p10, p11));
        // ---- O^T += V^T P^T: tiles of 16 head dimensions x 8 query rows ----
        {
          const int row = tw0 + (mi >> 1) * 8 + (lane & 7);
#pragma unroll
          for (int t = 0; t < D / 16; ++t) {
            const int cg = t * 2 + (mi & 1);
            uint32_t a[4];
            ldsm_x4_t(vb + (cg >> 3) * HALF_B + row * 128 + (((cg & 7) ^ (row & 7)) << 4), a[0], a[1], a[2], a[3]);
            mma16816(o[t], a, pb0, pb1);
          }
        }
      } else {
      // ---- S = Q K^T ----
      // (the k-steps of a tile go to CH independent accumulators: a chain of dependent MMAs is the
      // longest latency in the loop)
      constexpr int CH = (NT == 1) ? 4 : (NT <= 2 ? 2 : 1);
      float sc[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float part[CH][4];
#pragma unroll
        for (int c = 0; c < CH; ++c) part[c][0] = part[c][1] = part[c][2] = part[c][3] = 0.f;
        const int row = tw0 + nt * 8 + (lane & 7);
        if (nt * 8 < tw && tw0 + nt * 8 < rows) {  // warp-uniform: this 8-key tile is in my slice and holds keys
#pragma unroll
          for (int k2 = 0; k2 < KS / 2; ++k2) {
            const int cg = k2 * 4 + (lane >> 3);
            uint32_t b0, b1, b2, b3;
            ldsm_x4(kb + (cg >> 3) * HALF_B + row * 128 + (((cg & 7) ^ (row & 7)) << 4), b0, b1, b2, b3);
            mma16816(part[(2 * k2) % CH], qa[2 * k2], b0, b1);
            mma16816(part[(2 * k2 + 1) % CH], qa[2 * k2 + 1], b2, b3);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float t = part[0][e];
#pragma unroll
            for (int c = 1; c < CH; ++c) t += part[c][e];
            sc[nt][e] = t;
          }
        } else {
          sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = -INFINITY;
        }
      }
      // ---- scale, additive mask, visibility ----
      const int t_base = tok0 + tw0 + 2 * qc;  // key index of sc[0][0]
      const bool need_mask = (tw0 + tw > rows) || (tok0 + tw0 < kvs) || (tok0 + tw0 + tw > min(lim0, lim1));
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[nt][e] *= p.scale_log2;
      }
      if (p.mask) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int t = t_base + nt * 8 + (e & 1);
            const int sq = (e < 2) ? srow0 : srow1;
            if (t < tok0 + rows && sq < p.q_len) {
              const size_t off = (size_t)bcur * p.mask_sb + (size_t)(p.mask_rows == 1 ? 0 : sq) * p.kv.fixed_len + t;
              const float mv = p.mask_fp32 ? reinterpret_cast<const float*>(p.mask)[off]
                                           : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.mask)[off]);
              sc[nt][e] += mv * kLog2e;
            }
          }
      }
      if (need_mask) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int t = t_base + nt * 8 + (e & 1);
            const int lim = (e < 2) ? lim0 : lim1;
            if (t >= tok0 + rows || t < kvs || t >= lim) sc[nt][e] = -INFINITY;
          }
      }
      // ---- online softmax ----
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        mx0 = fmaxf(mx0, fmaxf(sc[nt][0], sc[nt][1]));
        mx1 = fmaxf(mx1, fmaxf(sc[nt][2], sc[nt][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
      const float a0 = (m0 == -INFINITY) ? 0.f : fast_exp2(m0 - n0);
      const float a1 = (m1 == -INFINITY) ? 0.f : fast_exp2(m1 - n1);
      const float e0 = (n0 == -INFINITY) ? 0.f : n0, e1 = (n1 == -INFINITY) ? 0.f : n1;
      m0 = n0;
      m1 = n1;
      l0 *= a0;
      l1 *= a1;
#pragma unroll
      for (int n = 0; n < ON; ++n) {
        o[n][0] *= a0;
        o[n][1] *= a0;
        o[n][2] *= a1;
        o[n][3] *= a1;
      }
      uint32_t pk[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const float p00 = fast_exp2(sc[nt][0] - e0), p01 = fast_exp2(sc[nt][1] - e0);
        const float p10 = fast_exp2(sc[nt][2] - e1), p11 = fast_exp2(sc[nt][3] - e1);
        l0 += p00 + p01;
        l1 += p10 + p11;
        pk[nt][0] = f2_to_bf2(p00, p01);
        pk[nt][1] = f2_to_bf2(p10, p11);
      }
      // ---- O += P V ----
      if constexpr (NT == 1) {
#pragma unroll
        for (int n4 = 0; n4 < ON / 4; ++n4) {
          const int row = tw0 + (lane & 7);
          const int cg = n4 * 4 + (lane >> 3);
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(vb + (cg >> 3) * HALF_B + row * 128 + (((cg & 7) ^ (row & 7)) << 4), b0, b1, b2, b3);
          mma1688(o[n4 * 4 + 0], pk[0][0], pk[0][1], b0);
          mma1688(o[n4 * 4 + 1], pk[0][0], pk[0][1], b1);
          mma1688(o[n4 * 4 + 2], pk[0][0], pk[0][1], b2);
          mma1688(o[n4 * 4 + 3], pk[0][0], pk[0][1], b3);
        }
      } else {
#pragma unroll
        for (int kb2 = 0; kb2 < NT / 2; ++kb2) {
          if (kb2 * 16 < tw && tw0 + kb2 * 16 < rows) {  // warp-uniform: skip 16-key blocks outside my slice
            const uint32_t a[4] = {pk[2 * kb2][0], pk[2 * kb2][1], pk[2 * kb2 + 1][0], pk[2 * kb2 + 1][1]};
            const int mi = lane >> 3;
            const int row = tw0 + kb2 * 16 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
            for (int n2 = 0; n2 < ON / 2; ++n2) {
              const int cg = n2 * 2 + (mi >> 1);
              uint32_t b0, b1, b2, b3;
              ldsm_x4_t(vb + (cg >> 3) * HALF_B + row * 128 + (((cg & 7) ^ (row & 7)) << 4), b0, b1, b2, b3);
              mma16816(o[2 * n2], a, b0, b1);
              mma16816(o[2 * n2 + 1], a, b2, b3);
            }
          }
        }
      }
      }  // row-major path
    }
    if (flags & 2) fin.last_part = (flags & 4) ? 1 : 0;
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);

    if (flags & 2) {
      // ================= end of a unit part: hand the result to the epilogue warp =================
      float lt0 = l0, lt1 = l1;
      if (tr) {  // a query row's keys sit in the 8 lanes with the same qc
#pragma unroll
        for (int o_ = 4; o_ < 32; o_ <<= 1) {
          lt0 += __shfl_xor_sync(0xffffffffu, lt0, o_);
          lt1 += __shfl_xor_sync(0xffffffffu, lt1, o_);
        }
      } else {
        lt0 += __shfl_xor_sync(0xffffffffu, lt0, 1);
        lt0 += __shfl_xor_sync(0xffffffffu, lt0, 2);
        lt1 += __shfl_xor_sync(0xffffffffu, lt1, 1);
        lt1 += __shfl_xor_sync(0xffffffffu, lt1, 2);
      }
      const int live = fin.live;
      const int row0 = mt * 16 + qr, row1 = row0 + 8;
      const int rs = n_parts_done % sp.n_res;
      float* rnum = reinterpret_cast<float*>(res + (size_t)rs * sp.res_slot_bytes);
      float* rM = rnum + p.live_max * D;
      float* rden = rM + p.live_max;
      bool ok_res = true;
      if (NS > 1) {
        // the NS token slices of each row meet in shared memory
        csync<CTHR>();  // every thread is done reading the merge buffer for the previous part
        float* wo = mg_o + (size_t)ns * p.live_max * sp.mg_stride;
        if (tr) {
          // transposed accumulators: o[t] = head dimensions 16 t + qr (+ 8) of query rows 2 qc, 2 qc + 1
          const int ra = 2 * qc, rb = ra + 1;
          if (ra < live) {
#pragma unroll
            for (int t = 0; t < D / 16; ++t) {
              wo[ra * sp.mg_stride + 16 * t + qr] = o[t][0];
              wo[ra * sp.mg_stride + 16 * t + qr + 8] = o[t][2];
            }
            if (qr == 0) {
              mg_m[ns * p.live_max + ra] = m0;
              mg_l[ns * p.live_max + ra] = lt0;
            }
          }
          if (rb < live) {
#pragma unroll
            for (int t = 0; t < D / 16; ++t) {
              wo[rb * sp.mg_stride + 16 * t + qr] = o[t][1];
              wo[rb * sp.mg_stride + 16 * t + qr + 8] = o[t][3];
            }
            if (qr == 0) {
              mg_m[ns * p.live_max + rb] = m1;
              mg_l[ns * p.live_max + rb] = lt1;
            }
          }
        } else {
        if (row0 < live) {
#pragma unroll
          for (int n = 0; n < ON; ++n)
            *reinterpret_cast<float2*>(wo + row0 * sp.mg_stride + n * 8 + 2 * qc) = make_float2(o[n][0], o[n][1]);
          if (qc == 0) {
            mg_m[ns * p.live_max + row0] = m0;
            mg_l[ns * p.live_max + row0] = lt0;
          }
        }
        if (row1 < live) {
#pragma unroll
          for (int n = 0; n < ON; ++n)
            *reinterpret_cast<float2*>(wo + row1 * sp.mg_stride + n * 8 + 2 * qc) = make_float2(o[n][2], o[n][3]);
          if (qc == 0) {
            mg_m[ns * p.live_max + row1] = m1;
            mg_l[ns * p.live_max + row1] = lt1;
          }
        }
        }  // row-major accumulators
        if (n_parts_done >= sp.n_res) ok_res = mbar_wait(&res_empty[rs], ((n_parts_done / sp.n_res) - 1) & 1, abort);
        csync<CTHR>();
        for (int oi = tid; oi < live * D; oi += CTHR) {
          const int row = oi / D, d = oi - row * D;
          float M = -INFINITY;
#pragma unroll
          for (int w = 0; w < NS; ++w) M = fmaxf(M, mg_m[w * p.live_max + row]);
          float num = 0.f, den = 0.f;
          if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < NS; ++w) {
              const float mw = mg_m[w * p.live_max + row];
              const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
              num += mg_o[((size_t)w * p.live_max + row) * sp.mg_stride + d] * f;
              den += mg_l[w * p.live_max + row] * f;
            }
          }
          rnum[oi] = num;
          if (d == 0) {
            rM[row] = M;
            rden[row] = den;
          }
        }
      } else {
        // one warp owns its 16 rows outright: registers go straight to the result slot
        if (n_parts_done >= sp.n_res) ok_res = mbar_wait(&res_empty[rs], ((n_parts_done / sp.n_res) - 1) & 1, abort);
        if (row0 < live) {
#pragma unroll
          for (int n = 0; n < ON; ++n)
            *reinterpret_cast<float2*>(rnum + row0 * D + n * 8 + 2 * qc) = make_float2(o[n][0], o[n][1]);
          if (qc == 0) {
            rM[row0] = m0;
            rden[row0] = lt0;
          }
        }
        if (row1 < live) {
#pragma unroll
          for (int n = 0; n < ON; ++n)
            *reinterpret_cast<float2*>(rnum + row1 * D + n * 8 + 2 * qc) = make_float2(o[n][2], o[n][3]);
          if (qc == 0) {
            rM[row1] = m1;
            rden[row1] = lt1;
          }
        }
      }
      if (!ok_res) {
        if (lane == 0) raise_status(p.kv.status, PACE_DEV_WAIT_TIMEOUT);
        return;
      }
      if (tid == 0) *reinterpret_cast<ResMeta*>(rden + p.live_max) = fin;
      __syncwarp();
      if (lane == 0) mbar_arrive(&res_full[rs]);  // release: the slot's contents are visible to the waiter
      ++n_parts_done;
      if (fin.last_part) {
        // nothing is left to stream: all eight warps take the result out (the epilogue warp only
        // wakes up to leave), which keeps the kernel's tail short
        csync<CTHR>();
        publish_part<D, MR, CTHR, false>(p, fin, rnum, rM, rden, tid, cta, misc);
      }
    }
    if (flags & 4) break;  // the CTA's last chunk (the short prologue gives the consumers no count)
  }
}

// ------------------------------- host side -------------------------------
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(ptr);
  });
  return fn;
}

// bf16 tensor seen as [c3][tiles][rows][D]; box = 64 columns x box_rows rows, 128-byte swizzle
int make_map(CUtensorMap* tm, const void* base, int D, int rows, uint64_t tiles, uint64_t c3, uint64_t c3_stride_elems,
             int box_rows) {
  EncodeFn fn = encode_fn();
  if (!fn) {
    set_cuda_error(cudaErrorNotSupported, "cuTensorMapEncodeTiled entry point");
    return PACE_ERR_CUDA;
  }
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)rows, tiles, c3};
  const cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)rows * D * 2, c3_stride_elems * 2};
  const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return PACE_ERR_CUDA;
  }
  return PACE_OK;
}

struct PoolMapEntry {
  const void* pages;
  int geom[6];
  CUtensorMap tm;      // boxes of one page (or 64 rows of a larger page)
  CUtensorMap tm_sub;  // boxes of 16 rows
};
std::mutex g_map_mu;
PoolMapEntry g_maps[16];
int g_n_maps = 0, g_next_map = 0;

int pool_map(const pace_kv_pool_t* pl, CUtensorMap* out, CUtensorMap* out_sub) {
  const int geom[6] = {pl->n_layers, pl->n_kv_heads, pl->head_dim, pl->page_tokens, pl->n_pages, 0};
  std::lock_guard<std::mutex> lk(g_map_mu);
  for (int i = 0; i < g_n_maps; ++i)
    if (g_maps[i].pages == pl->pages && memcmp(g_maps[i].geom, geom, sizeof(geom)) == 0) {
      *out = g_maps[i].tm;
      *out_sub = g_maps[i].tm_sub;
      return PACE_OK;
    }
  CUtensorMap tm, tm_sub;
  const uint64_t tiles = (uint64_t)pl->n_pages * pl->n_kv_heads;
  int rc = make_map(&tm, pl->pages, pl->head_dim, pl->page_tokens, tiles, (uint64_t)pl->n_layers * 2,
                    tiles * pl->page_tokens * pl->head_dim, pl->page_tokens <= kChunk ? pl->page_tokens : kChunk);
  if (rc != PACE_OK) return rc;
  rc = make_map(&tm_sub, pl->pages, pl->head_dim, pl->page_tokens, tiles, (uint64_t)pl->n_layers * 2,
                tiles * pl->page_tokens * pl->head_dim, pl->page_tokens < 16 ? pl->page_tokens : 16);
  if (rc != PACE_OK) return rc;
  PoolMapEntry& e = g_maps[g_next_map];
  g_next_map = (g_next_map + 1) % 16;
  if (g_n_maps < 16) ++g_n_maps;
  e.pages = pl->pages;
  memcpy(e.geom, geom, sizeof(geom));
  e.tm = tm;
  e.tm_sub = tm_sub;
  *out = tm;
  *out_sub = tm_sub;
  return PACE_OK;
}

int sm_count_m() {
  int dev = 0, n = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}

// Fewest query rows (tokens x grouped heads) for which a tile goes to the tcgen05 variant.
// At 33 rows and more (PARD verify: 9 tokens x 4 grouped heads = 36) a 128-row tile, three quarters of
// it padding, already beats the mma.sync kernel's 64-row tiles: the MMAs cost the softmax warps
// nothing.
constexpr int kUmmaMinRows = 33;

// What run_mma needs beyond the operands of the reference op: the pending row of a decode launch,
// the caller's limit on thread blocks, and what the stream note records about the launch.
struct MmaExtra {
  const void* k_pend = nullptr;
  const void* v_pend = nullptr;
  int64_t pend_sb = 0, pend_sh = 0;
  int max_ctas = 0;            // 0: one thread block per SM (two for the four-warp decode form)
  bool one_cta_per_sm = false; // decode: keep the eight-warp form
  bool no_early_kv = false;
  const void* pages = nullptr; // pool the launch reads (null: the dense form)
  int layer = -1;
  const CUtensorMap* tm_sub = nullptr;  // the pool seen in 16-row boxes (64-token pages only)
};

template <int D, int MT, int NS, bool UMMA = false>
int launch_mma(MmaParams& p, const CUtensorMap& tmK, const CUtensorMap& tmV, int grid, cudaStream_t stream,
               const MmaExtra& ex) {
  constexpr int MR = 16 * MT;
  constexpr int NW = UMMA ? 8 : MT * NS;
  const int n_items = p.batch * p.n_qt;
  p.live_max = p.G * p.q_len < MR ? p.G * p.q_len : MR;
  // two CTAs per SM (four consumer warps): 228 KB of shared memory less 1 KB the system keeps per CTA
  const int budget = NW == 4 ? kHalfSmemBudget : 227 * 1024;  // (227 KB: the most one CTA may ask for)
  int ns = kMaxStagesM;
  while (ns >= 2 && plan_smem(D, MT, NS, ns, p.live_max, p.batch, n_items, UMMA).total > budget) --ns;
  if (ns < 2) return PACE_ERR_UNSUPPORTED;
  p.n_stages = ns;
  const size_t smem_bytes = plan_smem(D, MT, NS, ns, p.live_max, p.batch, n_items, UMMA).total;
  // Early K/V streaming: only the short prologue of whole-unit decode has it, and only when this
  // library's newest launch on the stream was an attention launch (nothing wrote the pool since).
  p.early_kv = (!UMMA && MT == 1 && p.whole_units && !ex.no_early_kv && ex.pages && !p.q_lens &&
                !stream_note(stream).pool_written)
                   ? 1
                   : 0;
  static bool configured[16] = {};
  int dev = 0;
  PACE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 16 || !configured[dev]) {
    PACE_CUDA_TRY(cudaFuncSetAttribute(attn_mma_kernel<D, MT, NS, UMMA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       budget));
    PACE_CUDA_TRY(cudaFuncSetAttribute(attn_mma_kernel<D, MT, NS, UMMA>,
                                       cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    if (dev < 16) configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(threads_of(UMMA, NW));
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  p.sub_boxes = (ex.tm_sub && !UMMA && MT == 1 && p.pages_per_chunk == 1 && p.kv.page_tokens == kChunk) ? 1 : 0;
  PACE_CUDA_TRY(cudaLaunchKernelEx(&cfg, attn_mma_kernel<D, MT, NS, UMMA>, p, tmK, tmV, ex.tm_sub ? *ex.tm_sub : tmK));
  PACE_LAUNCH_CHECK("attn_mma_kernel");
  note_attention_launch(stream, /*uses_workspace=*/!p.whole_units, ex.pages, ex.layer, p.q);
  return PACE_OK;
}

}  // namespace

uint64_t mma_workspace_bytes(int n_q_heads, int n_kv_heads, int head_dim, int q_len) {
  const int G = n_q_heads / (n_kv_heads > 0 ? n_kv_heads : 1);
  const int M = G * q_len;
  const int MT = M >= 2 * 128 ? 16 : M >= kUmmaMinRows ? 8 : M <= 16 ? 1 : M <= 32 ? 2 : M <= 64 ? 4 : 8;
  const int ctas = (MT == 1 ? 2 : 1) * sm_count_m();  // decode runs two four-warp CTAs per SM
  return kWorkspaceCounterBytes + (uint64_t)ctas * 2 * (16 * MT) * (head_dim + 2) * sizeof(float) + 256;
}

// One launch per slice of the batch small enough for the shared-memory prefix array.
int run_mma(const KVView& kv, const CUtensorMap& tmK, const CUtensorMap& tmV, int c3_k, int c3_v, int batch,
            int n_q_heads, int q_len, const void* q, int64_t q_sb, int64_t q_sh, int64_t q_ss, void* out, int64_t o_sb,
            int64_t o_sh, int64_t o_ss, const int32_t* kv_start, const int32_t* q_lens, int causal, float scale,
            const void* mask, int mask_fp32, int mask_rows, int64_t mask_sb, void* workspace, uint64_t workspace_bytes,
            uint32_t flags, cudaStream_t stream, const MmaExtra& ex) {
  const int D = kv.head_dim, Hkv = kv.n_kv_heads;
  if (batch <= 0 || q_len <= 0) return PACE_OK;
  if (n_q_heads % Hkv) return PACE_ERR_INVALID;
  const int G = n_q_heads / Hkv;
  if (!q || !out || ((uintptr_t)q & 15) || (q_sb & 7) || (q_sh & 7) || (q_ss & 7)) return PACE_ERR_INVALID;
  if (((uintptr_t)out & 3) || (o_sb & 1) || (o_sh & 1) || (o_ss & 1)) return PACE_ERR_INVALID;  // bf16 pairs are stored
  if (!workspace || ((uintptr_t)workspace & 15)) return PACE_ERR_INVALID;
  const int M = G * q_len;
  // 128-row tiles on the 5th-generation tensor cores (no additive mask there; 16-byte output stores)
  const bool pend = (flags & PACE_ATTN_PENDING_ROW) != 0;
  if (pend) {
    // one pending row per sequence: a decode launch over the pool, on the mma.sync kernels
    if (q_len != 1 || !ex.pages || mask || M >= kUmmaMinRows) return PACE_ERR_UNSUPPORTED;
    if (!ex.k_pend || !ex.v_pend || ((uintptr_t)ex.k_pend & 15) || ((uintptr_t)ex.v_pend & 15) || (ex.pend_sb & 7) ||
        (ex.pend_sh & 7))
      return PACE_ERR_INVALID;
  }
  const bool umma = M >= kUmmaMinRows && !mask && !((uintptr_t)out & 15) && !(o_sb & 7) && !(o_sh & 7) && !(o_ss & 7);
  // two 128-row tiles per unit from 256 query rows on (chunked prefill): they share each K/V chunk fetched
  const bool wide = umma && M >= 2 * kUmmaRows;
  const int MT = umma ? (wide ? 16 : 8) : M <= 16 ? 1 : M <= 32 ? 2 : M <= 64 ? 4 : 8;
  const int MR = 16 * MT;
  int grid = sm_count_m();
  auto workspace_for = [&](int ctas) { return kWorkspaceCounterBytes + (uint64_t)ctas * 2 * MR * (D + 2) * sizeof(float); };
  // Decode: CTAs of four consumer warps, two per SM, when the workspace has room for their partial
  // records (the fixed scratch of pace_attn_decode_static has not).
  // ... and three ring stages fit beside the per-sequence arrays (they do up to a batch of about 80).
  const int live = G * q_len < MR ? G * q_len : MR;
  const int slice = batch < kMaxItems ? batch : kMaxItems;
  const bool half = MT == 1 && !ex.one_cta_per_sm && workspace_bytes >= workspace_for(2 * grid) &&
                    plan_smem(D, 1, 4, 3, live, slice, slice, false).total <= kHalfSmemBudget;
  if (half) grid *= 2;
  if (ex.max_ctas > 0 && ex.max_ctas < grid) grid = ex.max_ctas;  // the caller's share of the GPU
  if (workspace_bytes < workspace_for(grid)) return PACE_ERR_INVALID;

  MmaParams p;
  p.kv = kv;
  p.c3_k = c3_k;
  p.c3_v = c3_v;
  p.q_sb = q_sb;
  p.q_sh = q_sh;
  p.q_ss = q_ss;
  p.o_sb = o_sb;
  p.o_sh = o_sh;
  p.o_ss = o_ss;
  p.q_len = q_len;
  p.G = G;
  p.n_qt = (M + MR - 1) / MR;
  p.causal = causal;
  p.whole_units = (flags & PACE_ATTN_WHOLE_UNITS) ? 1 : 0;
  p.scale_log2 = (scale > 0.f ? scale : 1.0f / sqrtf((float)D)) * kLog2e;
  p.unit_count = reinterpret_cast<int32_t*>(workspace);
  p.parts = reinterpret_cast<float*>(static_cast<char*>(workspace) + kWorkspaceCounterBytes);
  p.mask = mask;
  p.mask_fp32 = mask_fp32;
  p.mask_rows = mask_rows;
  p.mask_sb = mask_sb;
  p.k_pend = pend ? (const __nv_bfloat16*)ex.k_pend : nullptr;
  p.v_pend = pend ? (const __nv_bfloat16*)ex.v_pend : nullptr;
  p.pend_sb = ex.pend_sb;
  p.pend_sh = ex.pend_sh;
  p.early_kv = 0;
  const int P = kv.page_tokens;
  const int HALVES = D / 64;
  if (P <= kChunk) {
    const int most = 16 / HALVES;  // one producer lane per (page, K|V, column block)
    p.pages_per_chunk = kChunk / P < most ? kChunk / P : most;
    p.chunks_per_page = 0;
    p.chunk_tokens = p.pages_per_chunk * P;
    p.box_rows = P;
  } else {
    p.pages_per_chunk = 0;
    p.chunks_per_page = (P + kChunk - 1) / kChunk;
    p.chunk_tokens = kChunk;
    p.box_rows = kChunk;
  }
  int per_launch = kMaxItems / p.n_qt;
  if (per_launch < 1) return PACE_ERR_UNSUPPORTED;
  if ((uint64_t)per_launch * p.n_qt * Hkv * sizeof(int32_t) > kWorkspaceCounterBytes)
    per_launch = (int)(kWorkspaceCounterBytes / sizeof(int32_t) / ((uint64_t)p.n_qt * Hkv));
  if (per_launch < 1) return PACE_ERR_UNSUPPORTED;
  for (int b0 = 0; b0 < batch; b0 += per_launch) {
    const int nb = batch - b0 < per_launch ? batch - b0 : per_launch;
    p.batch = nb;
    p.kv.seq_ids = kv.seq_ids ? kv.seq_ids + b0 : nullptr;
    p.kv.slot_base = kv.seq_ids ? 0 : kv.slot_base + b0;  // (slots that are not listed are the batch indices)
    p.q = (const __nv_bfloat16*)q + (size_t)b0 * q_sb;
    p.out = (__nv_bfloat16*)out + (size_t)b0 * o_sb;
    p.kv_start = kv_start ? kv_start + b0 : nullptr;
    p.q_lens = q_lens ? q_lens + b0 : nullptr;
    if (pend) {
      p.k_pend = (const __nv_bfloat16*)ex.k_pend + (size_t)b0 * ex.pend_sb;
      p.v_pend = (const __nv_bfloat16*)ex.v_pend + (size_t)b0 * ex.pend_sb;
    }
    int rc = PACE_ERR_UNSUPPORTED;
#define PACE_MMA_CASE(DD, MM, NN) \
  if (D == DD && MT == MM) rc = launch_mma<DD, MM, NN>(p, tmK, tmV, grid, stream, ex);
    if (umma && wide) {
      if (D == 128) rc = launch_mma<128, 16, 1, true>(p, tmK, tmV, grid, stream, ex);
      if (D == 64) rc = launch_mma<64, 16, 1, true>(p, tmK, tmV, grid, stream, ex);
    } else if (umma) {
      if (D == 128) rc = launch_mma<128, 8, 1, true>(p, tmK, tmV, grid, stream, ex);
      if (D == 64) rc = launch_mma<64, 8, 1, true>(p, tmK, tmV, grid, stream, ex);
    } else {
      if (half) {
        if (D == 128) rc = launch_mma<128, 1, 4>(p, tmK, tmV, grid, stream, ex);
        if (D == 64) rc = launch_mma<64, 1, 4>(p, tmK, tmV, grid, stream, ex);
      } else {
        PACE_MMA_CASE(128, 1, 8)
        PACE_MMA_CASE(64, 1, 8)
      }
      PACE_MMA_CASE(128, 2, 4)
      PACE_MMA_CASE(128, 4, 2)
      PACE_MMA_CASE(128, 8, 1)
      PACE_MMA_CASE(64, 2, 4)
      PACE_MMA_CASE(64, 4, 2)
      PACE_MMA_CASE(64, 8, 1)
    }
#undef PACE_MMA_CASE
    if (rc != PACE_OK) return rc;
  }
  return PACE_OK;
}

int run_mma_paged(const pace_attn_args_t* a, int causal, cudaStream_t stream) {
  if (!a || !a->pool || a->q_len < 1 || a->layer < 0 || a->layer >= a->pool->n_layers) return PACE_ERR_INVALID;
  if (a->batch > a->pool->max_seqs) return PACE_ERR_INVALID;
  CUtensorMap tm, tm_sub;
  const int rc = pool_map(a->pool, &tm, &tm_sub);
  if (rc != PACE_OK) return rc;
  const KVView kv = make_view(a->pool, a->layer, a->seq_ids);
  MmaExtra ex;
  if (a->flags & PACE_ATTN_PENDING_ROW) {
    ex.k_pend = a->k_pending;
    ex.v_pend = a->v_pending;
    ex.pend_sb = a->pending_stride_b;
    ex.pend_sh = a->pending_stride_h;
  }
  ex.max_ctas = a->max_ctas;
  ex.one_cta_per_sm = (a->flags & PACE_ATTN_ONE_CTA_PER_SM) != 0;
  ex.no_early_kv = (a->flags & PACE_ATTN_NO_EARLY_KV) != 0;
  ex.pages = a->pool->pages;
  ex.layer = a->layer;
  ex.tm_sub = &tm_sub;
  return run_mma(kv, tm, tm, a->layer * 2, a->layer * 2 + 1, a->batch, a->n_q_heads, a->q_len, a->q, a->q_stride_b,
                 a->q_stride_h, a->q_stride_s, a->out, a->o_stride_b, a->o_stride_h, a->o_stride_s, a->kv_start,
                 a->q_lens, causal, a->scale, nullptr, 0, 1, 0, a->workspace, a->workspace_bytes, a->flags, stream, ex);
}

}  // namespace pace

using namespace pace;

// ---------------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc on the path that runs a decode step: code
// inside a region that forbids allocation (a serving loop that has handed all of its memory to a
// fixed arena, a real-time thread, a process whose memory budget was frozen at start-up), or a
// plug-in loaded into an engine that owns every byte of the device.  pace_attn_decode needs a
// caller-provided workspace; this entry point instead keeps the scratch in a file-scope device
// array that every GPU loading the library holds until the process exits.
//
// kStaticScratchBytes bounds what it can serve (see the checks below); anything larger is refused
// with PACE_ERR_UNSUPPORTED.  All calls on a device share the one array, which still holds what
// the previous call left: the arrival counters the kernel needs at zero are cleared on the stream
// before every launch, and two calls that overlap on the GPU (different streams) race on it.
constexpr int kStaticMaxSMs = 192;
constexpr uint64_t kStaticPartBytes = (uint64_t)kStaticMaxSMs * 2 * 16 * (128 + 2) * sizeof(float);
constexpr uint64_t kStaticScratchBytes = kWorkspaceCounterBytes + kStaticPartBytes + 256;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace pace {
namespace {
// In host code `g_static_scratch` is only a handle for the runtime, not an address the GPU can
// use: the device address is asked for once per device, with that device current.
int static_scratch_ptr(void** out) {
  static void* ptrs[64] = {};
  static std::mutex mu;
  int dev = 0;
  PACE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return PACE_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lk(mu);
  if (!ptrs[dev]) {
    void* ptr = nullptr;
    PACE_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
    ptrs[dev] = ptr;
  }
  *out = ptrs[dev];
  return PACE_OK;
}
}  // namespace
}  // namespace pace

extern "C" int pace_attn_decode_static(const pace_attn_args_t* a, void* stream) {
  if (!a || !a->pool || a->q_len != 1 || a->batch < 0) return PACE_ERR_INVALID;
  const pace_kv_pool_t* pl = a->pool;
  if (pl->n_kv_heads <= 0 || a->n_q_heads % pl->n_kv_heads) return PACE_ERR_INVALID;
  const int G = a->n_q_heads / pl->n_kv_heads;
  // limits of the fixed scratch: one 16-row tile of grouped heads, counters for every (sequence, kv head)
  if (G > 16 || pl->head_dim > 128) return PACE_ERR_UNSUPPORTED;
  if ((uint64_t)a->batch * pl->n_kv_heads * sizeof(int32_t) > kWorkspaceCounterBytes) return PACE_ERR_UNSUPPORTED;
  if (sm_count_m() > kStaticMaxSMs) return PACE_ERR_UNSUPPORTED;
  if (a->layer < 0 || a->layer >= pl->n_layers || a->batch > pl->max_seqs) return PACE_ERR_INVALID;  // before the array is touched
  if (a->batch == 0) return PACE_OK;
  void* scratch = nullptr;
  const int rc = static_scratch_ptr(&scratch);  // first call on a device: resolves the array's device address
  if (rc != PACE_OK) return rc;
  PACE_CUDA_TRY(cudaMemsetAsync(scratch, 0, (size_t)a->batch * pl->n_kv_heads * sizeof(int32_t), (cudaStream_t)stream));
  pace_attn_args_t b = *a;
  b.workspace = scratch;
  b.workspace_bytes = kStaticScratchBytes;
  return run_mma_paged(&b, 1, (cudaStream_t)stream);
}

extern "C" int pace_attn_verify(const pace_attn_args_t* a, void* stream) {
  PACE_PROFILE("attn_multi_query", stream, "layer=%d batch=%d q_len=%d heads=%d", a ? a->layer : -1, a ? a->batch : 0,
               a ? a->q_len : 0, a ? a->n_q_heads : 0);
  return run_mma_paged(a, 1, (cudaStream_t)stream);
}
// (an alias: one kernel family serves every query length; the name is what a chunked-prefill caller looks for)
extern "C" int pace_attn_prefill(const pace_attn_args_t* a, void* stream) { return pace_attn_verify(a, stream); }

extern "C" int pace_attention_dense(const void* q, const void* k, const void* v, const void* mask,
                                    int32_t mask_is_fp32, int32_t mask_rows, void* out, int32_t B, int32_t N,
                                    int32_t Nkv, int32_t S, int32_t L, int32_t H, void* workspace,
                                    uint64_t workspace_bytes, void* stream) {
  if (!q || !k || !v || !out || B <= 0 || N <= 0 || Nkv <= 0 || S <= 0 || L <= 0) return PACE_ERR_INVALID;
  if (H != 64 && H != 128) return PACE_ERR_UNSUPPORTED;
  PACE_PROFILE("attention", stream, "q=[%d,%d,%d,%d] kv=[%d,%d,%d,%d] mask=%d", B, N, S, H, B, Nkv, L, H, mask ? 1 : 0);
  if (N % Nkv || (mask && mask_rows != 1 && mask_rows != S)) return PACE_ERR_INVALID;
  if (((uintptr_t)k & 15) || ((uintptr_t)v & 15)) return PACE_ERR_INVALID;
  KVView kv;
  kv.k = (const __nv_bfloat16*)k;
  kv.v = (const __nv_bfloat16*)v;
  kv.block_table = nullptr;
  kv.seq_ids = nullptr;
  kv.slot_base = 0;
  kv.seq_len = nullptr;
  kv.status = nullptr;
  kv.fixed_len = L;
  kv.page_tokens = L;
  kv.n_kv_heads = Nkv;
  kv.head_dim = H;
  kv.max_pages_per_seq = 1;
  kv.max_seqs = B;
  kv.n_pages = B;
  CUtensorMap tmK, tmV;
  const int box_rows = L <= kChunk ? L : kChunk;
  int rc = make_map(&tmK, k, H, L, (uint64_t)B * Nkv, 1, (uint64_t)B * Nkv * L * H, box_rows);
  if (rc != PACE_OK) return rc;
  rc = make_map(&tmV, v, H, L, (uint64_t)B * Nkv, 1, (uint64_t)B * Nkv * L * H, box_rows);
  if (rc != PACE_OK) return rc;
  return run_mma(kv, tmK, tmV, 0, 0, B, N, S, q, (int64_t)N * S * H, (int64_t)S * H, H, out, (int64_t)N * S * H,
                 (int64_t)S * H, H, nullptr, nullptr, /*causal=*/0, 0.f, mask, mask_is_fp32, mask_rows,
                 (int64_t)mask_rows * L, workspace, workspace_bytes, 0u, (cudaStream_t)stream, MmaExtra());
}
