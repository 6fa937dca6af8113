// GQA decode attention (one query token per sequence) over the paged KV pool.
//
// Replaces, for q_len == 1, the reference's four-primitive SDPA sequence
// (csrc/ops/kernels/attention_kernels.cpp:218-257) and the repeat_kv expansion
// in front of it (pace/llm/models/llama.py:152-158): every K/V byte is read from
// HBM exactly once and serves all G query heads of its KV head.
//
// Shape of the kernel (HBM-bound: 4 flop per byte at G = 4):
//   * persistent grid, one CTA per SM; the global sequence of K/V chunks
//     (all sequences x kv heads) is cut into equal contiguous ranges, one per
//     CTA, so every SM streams the same number of bytes whatever the lengths;
//   * one producer warp walks the block table and feeds a shared-memory ring
//     with TMA bulk copies (cp.async.bulk + mbarrier complete_tx), running ahead
//     across sequence boundaries;
//   * eight consumer warps; 8 lanes share a K/V row (16 bytes per lane per
//     load, conflict-free), 4 rows per warp step; QK^T and PV on CUDA cores
//     with packed fp32 FMAs, fp32 accumulation, warp-shuffle online softmax;
//   * a (sequence, kv head) unit cut by a range boundary leaves fp32 partials
//     in the workspace; the last CTA to arrive merges them (no CTA waits on
//     another).
#include <cfloat>
#include <cstdlib>

#include "common.cuh"

namespace pace {
namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;  // + producer warp
constexpr int kChunkRows = 64;                   // rows of K (and of V) per ring stage, at most
constexpr int kMaxStages = 12;
constexpr int kRowsPerStep = kConsumerWarps * 4;

struct StageMeta {  // written by the producer, read by every consumer
  int rows;         // valid rows in this chunk
  int tok0;         // token index of row 0
  int flags;        // bit0: first chunk of a unit part, bit1: last chunk of a unit part
  int unit;         // b * Hkv + h
  int kv_start;     // first visible token of the sequence
  int mode;         // 0: part covers the whole unit; 1: partial -> workspace slot 0; 2: slot 1
  int parts;        // CTAs sharing the unit
  int first_cta;    // first of them
  int first_slot;   // workspace slot the first of them uses
  int pad[7];
};
static_assert(sizeof(StageMeta) == 64, "StageMeta is one 64-byte line");

struct DecodeParams {
  KVView kv;
  const __nv_bfloat16* q;
  int64_t q_sb, q_sh;
  __nv_bfloat16* out;
  int64_t o_sb, o_sh;
  const int32_t* kv_start;
  int batch;
  float scale_log2;   // softmax scale * log2(e)
  float* parts;       // [gridDim.x][2][G * (D + 2)]
  int32_t* unit_count;  // [batch * Hkv], zero between launches
  int chunk_tokens;   // tokens covered by a full chunk
  int pages_per_chunk;  // > 0: a chunk is this many whole pages (page_tokens <= 64)
  int chunks_per_page;  // > 0: a page is cut into this many chunks (page_tokens > 64)
  int n_stages;
  int stage_bytes;
};

__device__ __forceinline__ int chunks_of(const DecodeParams& p, int len) {
  if (len <= 0) return 0;
  if (p.pages_per_chunk > 0) return (len + p.chunk_tokens - 1) / p.chunk_tokens;
  const int P = p.kv.page_tokens;
  const int full = len / P, rem = len - full * P;
  return full * p.chunks_per_page + (rem + kChunkRows - 1) / kChunkRows;
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); }

// Sum over the 8 lanes of a row group while distributing heads: afterwards lane j
// holds the total of head j * N / 8 (duplicated on 8 / N lanes).
template <int N, int MASK>
struct HeadReduce {
  static __device__ __forceinline__ float run(const float* v, int lane) {
    if constexpr (MASK == 0) {
      return v[0];
    } else if constexpr (N > 1) {
      const bool up = (lane & MASK) != 0;
      float w[N / 2];
#pragma unroll
      for (int i = 0; i < N / 2; ++i) {
        const float keep = up ? v[N / 2 + i] : v[i];
        const float send = up ? v[i] : v[N / 2 + i];
        w[i] = keep + __shfl_xor_sync(0xffffffffu, send, MASK);
      }
      return HeadReduce<N / 2, MASK / 2>::run(w, lane);
    } else {
      float w[1] = {v[0] + __shfl_xor_sync(0xffffffffu, v[0], MASK)};
      return HeadReduce<1, MASK / 2>::run(w, lane);
    }
  }
};

// Sum accumulators over the 4 row groups of a warp (lane bits 4 and 3) while
// distributing heads.  acc is [N][W] float2; result in the first heads_left rows.
template <int N, int W, int MASK>
struct AccReduce {
  static __device__ __forceinline__ void run(float2 (*acc)[W], int lane) {
    if constexpr (MASK >= 8) {
      if constexpr (N > 1) {
        const bool up = (lane & MASK) != 0;
#pragma unroll
        for (int i = 0; i < N / 2; ++i) {
#pragma unroll
          for (int e = 0; e < W; ++e) {
            const float2 keep = up ? acc[N / 2 + i][e] : acc[i][e];
            const float2 send = up ? acc[i][e] : acc[N / 2 + i][e];
            float2 r;
            r.x = keep.x + __shfl_xor_sync(0xffffffffu, send.x, MASK);
            r.y = keep.y + __shfl_xor_sync(0xffffffffu, send.y, MASK);
            acc[i][e] = r;
          }
        }
        AccReduce<N / 2, W, MASK / 2>::run(acc, lane);
      } else {
#pragma unroll
        for (int e = 0; e < W; ++e) {
          acc[0][e].x += __shfl_xor_sync(0xffffffffu, acc[0][e].x, MASK);
          acc[0][e].y += __shfl_xor_sync(0xffffffffu, acc[0][e].y, MASK);
        }
        AccReduce<1, W, MASK / 2>::run(acc, lane);
      }
    }
  }
};

template <int D, int G>
__global__ void __launch_bounds__(kThreads, 1) attn_decode_kernel(const DecodeParams p) {
  constexpr int DPL = D / 8;       // dims per lane
  constexpr int VEC = DPL / 8;     // 16-byte loads per lane per row
  constexpr int W = DPL / 2;       // float2 per lane per head
  constexpr int HPL = G >= 4 ? G / 4 : 1;  // heads a lane owns after the cross-group reduction
  constexpr int REC = G * (D + 2);  // floats in one partial record

  extern __shared__ __align__(1024) unsigned char smem[];
  // layout: [n_stages][K chunk | V chunk | Q (G rows) | StageMeta] | barriers | merge | prefix
  const int n_stages = p.n_stages;
  const int kv_bytes = kChunkRows * D * 2;  // one K (or V) chunk slot
  unsigned char* stage_base = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)n_stages * p.stage_bytes);
  uint64_t* empty_bar = full_bar + kMaxStages;
  float* merge_acc = reinterpret_cast<float*>(empty_bar + kMaxStages);  // [warps][G][D]
  float* merge_m = merge_acc + kConsumerWarps * G * D;                  // [warps][G]
  float* merge_l = merge_m + kConsumerWarps * G;                        // [warps][G]
  int* misc = reinterpret_cast<int*>(merge_l + kConsumerWarps * G);     // [0] abort, [1] is_last
  int* prefix = misc + 8;                                               // [batch + 1]

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int Hkv = p.kv.n_kv_heads;
  const int P = p.kv.page_tokens;

  // ---- prologue: barriers, per-sequence chunk counts, exclusive prefix ----
  // (the pool's status word is asked for now and looked at behind the loads of the lengths: a launch on
  // a pool where an earlier launch ran out of patience does nothing)
  const int status_word = tid == kThreads - 1 ? load_status_word(p.kv.status) : 0;
  if (tid == 0) {
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kConsumerWarps);
    }
    misc[0] = 0;  // the CTA's abort flag
    misc[1] = 0;
    fence_mbar_init();
  }
  volatile int* abort = misc;
  for (int b = tid; b < p.batch; b += kThreads) {
    const int slot = view_slot(p.kv, b);
    prefix[b + 1] = slot < 0 ? 0 : chunks_of(p, view_len(p.kv, slot)) * Hkv;
  }
  if (__syncthreads_or(pool_gave_up(status_word))) return;
  if (warp == 0) {  // inclusive scan, 32 entries per round
    int carry = 0;
    for (int base = 0; base < p.batch; base += 32) {
      const int i = base + lane;
      int v = i < p.batch ? prefix[i + 1] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
      }
      if (i < p.batch) prefix[i + 1] = v + carry;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
    if (lane == 0) prefix[0] = 0;
  }
  __syncthreads();
  const long long T = prefix[p.batch];
  // with fewer chunks than CTAs only the first T CTAs work, so that the CTAs sharing a
  // unit are always consecutive
  const int NC = (long long)gridDim.x < T ? (int)gridDim.x : (int)T;
  const int cta = blockIdx.x;
  const long long x0 = cta < NC ? T * cta / NC : 0, x1 = cta < NC ? T * (cta + 1) / NC : 0;

  // sequences with nothing cached get zeros (no chunk will ever visit them)
  for (int u = cta; u < p.batch * Hkv; u += gridDim.x) {
    const int b = u / Hkv, h = u - b * Hkv;
    if (prefix[b + 1] == prefix[b]) {
      for (int o = tid; o < G * D; o += kThreads) {
        const int hq = h * G + o / D;
        p.out[(size_t)b * p.o_sb + (size_t)hq * p.o_sh + (o % D)] = __float2bfloat16(0.f);
      }
    }
  }
  if (x1 <= x0) return;
  const int n_my = (int)(x1 - x0);

  if (warp == kConsumerWarps) {
    // =========================== producer warp ============================
    // Everything that costs (divisions, table walks, the partition arithmetic) is done once
    // per unit part; the per-chunk loop is a handful of integer operations, one prefetched
    // page-id load and the copies.
    int lo = 0, hi = p.batch - 1;
    while (lo < hi) {  // largest b with prefix[b] <= x0
      const int mid = (lo + hi + 1) >> 1;
      if ((long long)prefix[mid] <= x0) lo = mid; else hi = mid - 1;
    }
    int b = lo;
    int nch = (prefix[b + 1] - prefix[b]) / Hkv;
    int h = (int)((x0 - prefix[b]) / nch);
    int j = (int)((x0 - prefix[b]) - (long long)h * nch);
    const bool whole_pages = p.pages_per_chunk > 0;
    // this lane's copy: K or V of page `pi` of the chunk (whole-page mode) or of the chunk's one page
    const int pi = whole_pages ? (lane >> 1) : 0;
    const int is_v = lane & 1;
    const bool copier = whole_pages ? (lane < 2 * p.pages_per_chunk) : (lane < 2);
    const __nv_bfloat16* src_base = is_v ? p.kv.v : p.kv.k;
    PageWindow pw;
    const int win_step = whole_pages ? (32 / p.pages_per_chunk) * p.pages_per_chunk : 32;
    bool ok = true;
    int i = 0, issued = 0;
    while (i < n_my && ok) {
      // ------------------------------ unit part ------------------------------
      const int slot = view_slot(p.kv, b);
      const int len = view_len(p.kv, slot);
      const int kvs = p.kv_start ? p.kv_start[b] : 0;
      const int j_end = min(nch, j + (n_my - i));
      // how the part is finished: whole unit here, or a partial record for the last arriver
      int mode = 0, parts = 1, first_cta = cta, first_slot = 0;
      {
        const long long ub = (long long)prefix[b] + (long long)h * nch, ue = ub + nch;
        if (ub < x0 || ue > x1) {
          first_cta = ub >= x0 ? cta : (int)(((ub + 1) * NC + T - 1) / T) - 1;
          const int last_cta = ue <= x1 ? cta : (int)((ue * NC + T - 1) / T) - 1;
          parts = last_cta - first_cta + 1;
          first_slot = (ub >= x0 ? x0 : T * first_cta / NC) == ub ? 0 : 1;
          mode = (cta == first_cta) ? (first_slot ? 2 : 1) : 1;
        }
      }
      // chunk -> (first logical page, first row): incremental from here on
      int lp, row0;
      if (whole_pages) {
        lp = j * p.pages_per_chunk;
        row0 = 0;
      } else {
        lp = j / p.chunks_per_page;
        row0 = (j - lp * p.chunks_per_page) * kChunkRows;
      }
      pw.start(p.kv, slot, lp, win_step, lane);
      for (bool first = true; j < j_end; ++j, ++i, first = false) {
        // prefetch the next chunk's page id before blocking on the ring
        int lp_n = lp, row0_n = row0;
        if (whole_pages) {
          lp_n = lp + p.pages_per_chunk;
        } else {
          row0_n = row0 + kChunkRows;
          if (row0_n >= P) { row0_n = 0; lp_n = lp + 1; }
        }
        const int s = i % n_stages;
        if (i >= n_stages && !mbar_wait(&empty_bar[s], ((i / n_stages) - 1) & 1, abort)) { ok = false; break; }
        const int tok0 = whole_pages ? j * p.chunk_tokens : lp * P + row0;
        const int rows = whole_pages ? min(p.chunk_tokens, len - tok0) : min(min(kChunkRows, P - row0), len - tok0);
        const int my_rows = whole_pages ? max(0, min(P, rows - pi * P)) : rows;
        const bool last = (j == j_end - 1);
        unsigned char* st = stage_base + (size_t)s * p.stage_bytes;
        if (lane == 0) {
          StageMeta* m = reinterpret_cast<StageMeta*>(st + 2 * kv_bytes + G * D * 2);
          m->rows = rows;
          m->tok0 = tok0;
          m->flags = (first ? 1 : 0) | (last ? 2 : 0);
          m->kv_start = kvs;
          if (last) {
            m->unit = b * Hkv + h;
            m->mode = mode;
            m->parts = parts;
            m->first_cta = first_cta;
            m->first_slot = first_slot;
          }
          mbar_arrive_expect_tx(&full_bar[s], 2u * rows * D * 2u + (first ? G * D * 2u : 0u));
        }
        __syncwarp();
        bool page_bad = false;
        const int pg = pw.get(lp + pi, lp, lane);
        if (copier && my_rows > 0) {
          if (pg < 0) {
            page_bad = true;
          } else {
            const __nv_bfloat16* src = src_base + view_row_offset(p.kv, pg, h, row0);
            unsigned char* dst = st + (is_v ? kv_bytes : 0) + (size_t)pi * P * D * 2;
            bulk_g2s(dst, src, (uint32_t)my_rows * D * 2u, &full_bar[s]);
          }
        }
        if (first && lane < G) {
          const __nv_bfloat16* src = p.q + (size_t)b * p.q_sb + (size_t)(h * G + lane) * p.q_sh;
          bulk_g2s(st + 2 * kv_bytes + lane * D * 2, src, D * 2u, &full_bar[s]);
        }
        if (__any_sync(0xffffffffu, page_bad)) {
          if (lane == 0) raise_status(p.kv.status, PACE_DEV_BAD_INDEX);
          ok = false;  // the consumers' bounded wait on this stage gives up
          break;
        }
        ++issued;
        lp = lp_n;
        row0 = row0_n;
      }
      if (!ok) break;
      // ---- next unit ----
      j = 0;
      if (++h == Hkv) {
        h = 0;
        ++b;
        while (b < p.batch && prefix[b + 1] == prefix[b]) ++b;
        if (b >= p.batch) break;
        nch = (prefix[b + 1] - prefix[b]) / Hkv;
      }
    }
    if (!ok && lane == 0) {
      misc[0] = 1;
      raise_status(p.kv.status, PACE_DEV_WAIT_TIMEOUT);
      // let copies already in flight land before the CTA's shared memory is released
      const int from = issued > n_stages ? issued - n_stages : 0;
      for (int k = from; k < issued; ++k) mbar_wait(&full_bar[k % n_stages], (k / n_stages) & 1);
    }
    return;
  }

  // ============================= consumer warps =============================
  const int g = lane >> 3;         // row group within the warp
  const int j8 = lane & 7;         // position within the row group
  const int my_head = j8 * G / 8;  // head whose score this lane holds after HeadReduce
  float2 q2[G][W];
  float2 acc[G][W];
  float m_run = -INFINITY, l_run = 0.f;
#pragma unroll
  for (int hh = 0; hh < G; ++hh)
#pragma unroll
    for (int e = 0; e < W; ++e) {
      acc[hh][e] = make_float2(0.f, 0.f);
      q2[hh][e] = make_float2(0.f, 0.f);
    }

  for (int i = 0; i < n_my; ++i) {
    const int s = i % n_stages;
    if (!mbar_wait(&full_bar[s], (i / n_stages) & 1, abort)) {
      if (lane == 0) raise_status(p.kv.status, PACE_DEV_WAIT_TIMEOUT);
      return;  // every consumer warp times out on the same stage; nobody is left waiting on us
    }
    const unsigned char* st = stage_base + (size_t)s * p.stage_bytes;
    const StageMeta* meta = reinterpret_cast<const StageMeta*>(st + 2 * kv_bytes + G * D * 2);
    const int rows = meta->rows, tok0 = meta->tok0, flags = meta->flags, kvs = meta->kv_start;

    if (flags & 1) {  // new unit part: fetch q, reset the running state
      const uint4* qs = reinterpret_cast<const uint4*>(st + 2 * kv_bytes);
#pragma unroll
      for (int hh = 0; hh < G; ++hh)
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          const uint4 w4 = qs[hh * (D / 8) + v * 8 + j8];
          const uint32_t ws[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float2 f = bf2_to_f2(ws[e]);
            f.x *= p.scale_log2;
            f.y *= p.scale_log2;
            q2[hh][v * 4 + e] = f;
          }
        }
      m_run = -INFINITY;
      l_run = 0.f;
#pragma unroll
      for (int hh = 0; hh < G; ++hh)
#pragma unroll
        for (int e = 0; e < W; ++e) acc[hh][e] = make_float2(0.f, 0.f);
    }

    // ---- scores: up to two row steps per chunk ----
    const uint4* Ks = reinterpret_cast<const uint4*>(st);
    const uint4* Vs = reinterpret_cast<const uint4*>(st + kv_bytes);
    float sc[2];
    bool valid[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int r = t * kRowsPerStep + warp * 4 + g;
      valid[t] = (r < rows) && (tok0 + r >= kvs);
      float part[G];
#pragma unroll
      for (int hh = 0; hh < G; ++hh) part[hh] = 0.f;
      if (t * kRowsPerStep < rows) {  // warp-uniform: skip the second step of short chunks
        if (valid[t]) {
          float2 d2[G];
#pragma unroll
          for (int hh = 0; hh < G; ++hh) d2[hh] = make_float2(0.f, 0.f);
#pragma unroll
          for (int v = 0; v < VEC; ++v) {
            const uint4 w4 = Ks[r * (D / 8) + v * 8 + j8];
            const uint32_t ws[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 kf = bf2_to_f2(ws[e]);
#pragma unroll
              for (int hh = 0; hh < G; ++hh) d2[hh] = __ffma2_rn(kf, q2[hh][v * 4 + e], d2[hh]);
            }
          }
#pragma unroll
          for (int hh = 0; hh < G; ++hh) part[hh] = d2[hh].x + d2[hh].y;
        }
        const float tot = HeadReduce<G, 4>::run(part, lane);
        sc[t] = valid[t] ? tot : -INFINITY;
      } else {
        sc[t] = -INFINITY;
      }
    }
    // ---- online softmax update (per head, shared by the whole warp) ----
    float cm = fmaxf(sc[0], sc[1]);
    cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, 8));
    cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, 16));
    const float m_new = fmaxf(m_run, cm);
    if (__any_sync(0xffffffffu, m_new > m_run)) {
      const float alpha = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_new);
      l_run *= alpha;
#pragma unroll
      for (int hh = 0; hh < G; ++hh) {
        const float a = __shfl_sync(0xffffffffu, alpha, hh * (8 / G));
        const float2 a2 = make_float2(a, a);
#pragma unroll
        for (int e = 0; e < W; ++e) acc[hh][e] = __fmul2_rn(acc[hh][e], a2);
      }
      m_run = m_new;
    }
    float pr[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      pr[t] = (sc[t] == -INFINITY) ? 0.f : fast_exp2(sc[t] - m_run);
      l_run += pr[t];
    }
    // ---- P.V ----
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      if (t * kRowsPerStep < rows) {
        float ph[G];
#pragma unroll
        for (int hh = 0; hh < G; ++hh) ph[hh] = __shfl_sync(0xffffffffu, pr[t], (lane & 24) | (hh * (8 / G)));
        if (valid[t]) {
          const int r = t * kRowsPerStep + warp * 4 + g;
#pragma unroll
          for (int v = 0; v < VEC; ++v) {
            const uint4 w4 = Vs[r * (D / 8) + v * 8 + j8];
            const uint32_t ws[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 vf = bf2_to_f2(ws[e]);
#pragma unroll
              for (int hh = 0; hh < G; ++hh)
                acc[hh][v * 4 + e] = __ffma2_rn(vf, make_float2(ph[hh], ph[hh]), acc[hh][v * 4 + e]);
            }
          }
        }
      }
    }
    // meta fields needed after the stage is released
    const int unit = meta->unit, mode = meta->mode, parts = meta->parts, first_cta = meta->first_cta,
              first_slot = meta->first_slot;
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);

    if (flags & 2) {
      // =================== end of a unit part: merge the warps ===================
      float l_tot = l_run;
      l_tot += __shfl_xor_sync(0xffffffffu, l_tot, 8);
      l_tot += __shfl_xor_sync(0xffffffffu, l_tot, 16);
      AccReduce<G, W, 16>::run(acc, lane);
      // lane (g, j8) now owns HPL heads starting at head0, its DPL dims
      const int head0 = (G >= 4) ? g * (G / 4) : (G == 2 ? (g >> 1) : 0);
      const bool writer = (G >= 4) ? true : (G == 2 ? ((g & 1) == 0) : (g == 0));
      if (writer) {
#pragma unroll
        for (int hh = 0; hh < HPL; ++hh)
#pragma unroll
          for (int v = 0; v < VEC; ++v) {
            float4* dst = reinterpret_cast<float4*>(merge_acc + ((size_t)warp * G + head0 + hh) * D + (v * 8 + j8) * 8);
            dst[0] = make_float4(acc[hh][v * 4 + 0].x, acc[hh][v * 4 + 0].y, acc[hh][v * 4 + 1].x, acc[hh][v * 4 + 1].y);
            dst[1] = make_float4(acc[hh][v * 4 + 2].x, acc[hh][v * 4 + 2].y, acc[hh][v * 4 + 3].x, acc[hh][v * 4 + 3].y);
          }
      }
      if (g == 0 && (j8 % (8 / G)) == 0) {
        merge_m[warp * G + my_head] = m_run;
        merge_l[warp * G + my_head] = l_tot;
      }
      consumer_sync();
      const int b = unit / Hkv, h = unit - b * Hkv;
      float* rec = p.parts + ((size_t)cta * 2 + (mode == 2 ? 1 : 0)) * REC;
      for (int o = tid; o < G * D; o += kConsumerThreads) {
        const int hh = o / D, d = o - hh * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) M = fmaxf(M, merge_m[w * G + hh]);
        float num = 0.f, den = 0.f;
        if (M != -INFINITY) {
#pragma unroll
          for (int w = 0; w < kConsumerWarps; ++w) {
            const float mw = merge_m[w * G + hh];
            const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
            num += merge_acc[((size_t)w * G + hh) * D + d] * f;
            den += merge_l[w * G + hh] * f;
          }
        }
        if (mode == 0) {
          const float r = den > 0.f ? num / den : 0.f;
          p.out[(size_t)b * p.o_sb + (size_t)(h * G + hh) * p.o_sh + d] = __float2bfloat16(r);
        } else {
          rec[hh * D + d] = num;
          if (d == 0) {
            rec[G * D + hh] = M;
            rec[G * D + G + hh] = den;
          }
        }
      }
      if (mode != 0) {
        __threadfence();
        consumer_sync();
        if (tid == 0) {
          const int old = atomicAdd(&p.unit_count[unit], 1);
          misc[1] = (old == parts - 1);
          if (old == parts - 1) p.unit_count[unit] = 0;  // ready for the next launch
        }
        consumer_sync();
        if (misc[1]) {
          __threadfence();
          for (int o = tid; o < G * D; o += kConsumerThreads) {
            const int hh = o / D, d = o - hh * D;
            float M = -INFINITY;
            for (int c = 0; c < parts; ++c) {
              const float* r = p.parts + ((size_t)(first_cta + c) * 2 + (c == 0 ? first_slot : 0)) * REC;
              M = fmaxf(M, __ldcg(r + G * D + hh));
            }
            float num = 0.f, den = 0.f;
            if (M != -INFINITY) {
              for (int c = 0; c < parts; ++c) {
                const float* r = p.parts + ((size_t)(first_cta + c) * 2 + (c == 0 ? first_slot : 0)) * REC;
                const float mc = __ldcg(r + G * D + hh);
                const float f = (mc == -INFINITY) ? 0.f : fast_exp2(mc - M);
                num += __ldcg(r + hh * D + d) * f;
                den += __ldcg(r + G * D + G + hh) * f;
              }
            }
            const float res = den > 0.f ? num / den : 0.f;
            p.out[(size_t)b * p.o_sb + (size_t)(h * G + hh) * p.o_sh + d] = __float2bfloat16(res);
          }
        }
      }
      consumer_sync();  // merge buffers may be reused by the next unit part
    }
  }
}

template <int D, int G>
int launch_decode(const DecodeParams& p, int grid, size_t smem_bytes, cudaStream_t stream) {
  static bool configured[16] = {};
  int dev = 0;
  PACE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 16 && !configured[dev]) {
    PACE_CUDA_TRY(cudaFuncSetAttribute(attn_decode_kernel<D, G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       220 * 1024));
    configured[dev] = true;
  } else if (dev >= 16) {
    PACE_CUDA_TRY(cudaFuncSetAttribute(attn_decode_kernel<D, G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       220 * 1024));
  }
  attn_decode_kernel<D, G><<<grid, kThreads, smem_bytes, stream>>>(p);
  PACE_LAUNCH_CHECK("attn_decode_kernel");
  return PACE_OK;
}

int sm_count() {
  static int cached[16] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev < 16 && cached[dev]) return cached[dev];
  int n = 148;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (dev < 16) cached[dev] = n;
  return n;
}

}  // namespace

// Shared by the paged and the dense entry points.
int run_decode(const KVView& kv, int batch, int n_q_heads, const void* q, int64_t q_sb, int64_t q_sh, void* out,
               int64_t o_sb, int64_t o_sh, const int32_t* kv_start, float scale, void* workspace,
               uint64_t workspace_bytes, int max_ctas, cudaStream_t stream) {
  const int D = kv.head_dim, Hkv = kv.n_kv_heads;
  if (batch <= 0) return PACE_OK;
  if (n_q_heads % Hkv) return PACE_ERR_INVALID;
  const int G = n_q_heads / Hkv;
  if (!q || !out || ((uintptr_t)q & 15) || (q_sb & 7) || (q_sh & 7)) return PACE_ERR_INVALID;
  if (batch > 8192) return PACE_ERR_UNSUPPORTED;  // the prefix array lives in shared memory
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;  // the caller's share of the GPU
  const uint64_t rec = (uint64_t)G * (D + 2) * sizeof(float);
  if (!workspace || ((uintptr_t)workspace & 15)) return PACE_ERR_INVALID;

  DecodeParams p;
  p.kv = kv;
  p.q = (const __nv_bfloat16*)q;
  p.q_sb = q_sb;
  p.q_sh = q_sh;
  p.out = (__nv_bfloat16*)out;
  p.o_sb = o_sb;
  p.o_sh = o_sh;
  p.kv_start = kv_start;
  p.batch = batch;
  p.scale_log2 = (scale > 0.f ? scale : 1.0f / sqrtf((float)D)) * kLog2e;
  // The arrival counters must read zero at every launch.  They sit in a region of FIXED size at
  // the head of the workspace, whatever the batch, so that no launch ever stores anything else
  // there; each counter is put back to zero by the CTA that consumes it.
  p.unit_count = reinterpret_cast<int32_t*>(workspace);
  if ((uint64_t)batch * Hkv * sizeof(int32_t) > kWorkspaceCounterBytes) return PACE_ERR_UNSUPPORTED;
  if (workspace_bytes < kWorkspaceCounterBytes + (uint64_t)grid * 2 * rec) return PACE_ERR_INVALID;
  p.parts = reinterpret_cast<float*>(static_cast<char*>(workspace) + kWorkspaceCounterBytes);
  const int P = kv.page_tokens;
  if (P <= kChunkRows) {
    p.pages_per_chunk = kChunkRows / P < 16 ? kChunkRows / P : 16;  // 2 copies per page, one per producer lane
    p.chunks_per_page = 0;
    p.chunk_tokens = p.pages_per_chunk * P;
  } else {
    p.pages_per_chunk = 0;
    p.chunks_per_page = (P + kChunkRows - 1) / kChunkRows;
    p.chunk_tokens = kChunkRows;
  }
  p.stage_bytes = 2 * kChunkRows * D * 2 + G * D * 2 + (int)sizeof(StageMeta);
  const size_t fixed = 2 * kMaxStages * sizeof(uint64_t) + (size_t)kConsumerWarps * G * (D + 2) * sizeof(float) +
                       8 * sizeof(int) + (size_t)(batch + 1) * sizeof(int) + 64;
  const size_t budget = 216 * 1024;
  if (fixed + 2 * (size_t)p.stage_bytes > budget) return PACE_ERR_UNSUPPORTED;
  int ns = (int)((budget - fixed) / p.stage_bytes);
  if (ns > kMaxStages) ns = kMaxStages;
  p.n_stages = ns;
  const size_t smem_bytes = (size_t)ns * p.stage_bytes + fixed;

#define PACE_DECODE_CASE(DD, GG) \
  if (D == DD && G == GG) return launch_decode<DD, GG>(p, grid, smem_bytes, stream);
  PACE_DECODE_CASE(128, 1)
  PACE_DECODE_CASE(128, 2)
  PACE_DECODE_CASE(128, 4)
  PACE_DECODE_CASE(128, 8)
  PACE_DECODE_CASE(64, 1)
  PACE_DECODE_CASE(64, 2)
  PACE_DECODE_CASE(64, 4)
  PACE_DECODE_CASE(64, 8)
#undef PACE_DECODE_CASE
  return PACE_ERR_UNSUPPORTED;
}

uint64_t decode_workspace_bytes(int batch, int n_q_heads, int n_kv_heads, int head_dim) {
  const int G = n_q_heads / (n_kv_heads > 0 ? n_kv_heads : 1);
  const uint64_t rec = (uint64_t)G * (head_dim + 2) * sizeof(float);
  (void)batch;
  return kWorkspaceCounterBytes + (uint64_t)sm_count() * 2 * rec + 256;
}

}  // namespace pace

namespace pace {
int decode_cuda_cores(const pace_attn_args_t* a, void* stream) {
  if (!a || !a->pool || a->q_len != 1 || a->layer < 0 || a->layer >= a->pool->n_layers) return PACE_ERR_INVALID;
  if (a->batch > a->pool->max_seqs) return PACE_ERR_INVALID;
  const KVView kv = make_view(a->pool, a->layer, a->seq_ids);
  return run_decode(kv, a->batch, a->n_q_heads, a->q, a->q_stride_b, a->q_stride_h, a->out, a->o_stride_b,
                    a->o_stride_h, a->kv_start, a->scale, a->workspace, a->workspace_bytes, a->max_ctas,
                    (cudaStream_t)stream);
}
}  // namespace pace

extern "C" int pace_attn_decode_cuda_cores(const pace_attn_args_t* a, void* stream) {
  if (a && (a->flags & PACE_ATTN_PENDING_ROW)) return PACE_ERR_UNSUPPORTED;  // the tensor-core kernels take pending rows
  return pace::decode_cuda_cores(a, stream);
}
