// Device-resident paged KV pool: allocator, block tables, append / rollback /
// beam-gather kernels and their C ABI.
//
// Stands in for the reference's per-layer torch buffers and Python bookkeeping
// (pace/llm/cache.py:126-400).  All state lives in device memory and is mutated
// by stream-ordered kernels; the host never copies a table.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace pace {

static thread_local char g_err[512] = "";
void set_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_err, sizeof(g_err), "%s: %s (%s)", where, cudaGetErrorName(e), cudaGetErrorString(e));
}

namespace {

constexpr int kCounterFree = 0;    // number of free pages
constexpr int kCounterTicket = 8;  // + layer: append kernels of that layer, blocks finished (appends to
                                   // different layers may overlap on the GPU, each needs its own count)
constexpr int kCounterShared = 2;  // set by a beam gather: pages may have more than one owner

__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct MetaLayout {
  size_t block_table, seq_len, seq_pages, page_ref, free_stack, counters, status, table_tmp, total;
};

MetaLayout meta_layout(const pace_kv_pool_t* g) {
  MetaLayout m;
  size_t off = 0;
  auto take = [&](size_t n_int32) {
    size_t o = off;
    off = align_up(off + n_int32 * sizeof(int32_t), 256);
    return o;
  };
  const size_t S = g->max_seqs, MP = g->max_pages_per_seq, L = g->n_layers, NP = g->n_pages;
  m.block_table = take(S * MP);
  m.seq_len = take(L * S);
  m.seq_pages = take(S);
  m.page_ref = take(NP);
  m.free_stack = take(NP);
  m.counters = take(kCounterTicket + L);
  m.status = take(4);
  m.table_tmp = take(S * (MP + 4) + L * S);
  m.total = off;
  return m;
}

bool geometry_ok(const pace_kv_pool_t* g) {
  if (!g) return false;
  if (g->n_layers <= 0 || g->n_kv_heads <= 0 || g->page_tokens <= 0 || g->n_pages <= 0 || g->max_seqs <= 0 ||
      g->max_pages_per_seq <= 0)
    return false;
  if (g->head_dim != 64 && g->head_dim != 128) return false;
  return true;
}

// ---------------------------------------------------------------------------
// kernels
// ---------------------------------------------------------------------------
__device__ __forceinline__ int pop_page(const pace_kv_pool_t& p) {
  int idx = atomicSub(&p.counters[kCounterFree], 1) - 1;
  if (idx < 0) {
    atomicAdd(&p.counters[kCounterFree], 1);
    return -1;
  }
  return p.free_stack[idx];
}
__device__ __forceinline__ void push_page(const pace_kv_pool_t& p, int page) {
  int idx = atomicAdd(&p.counters[kCounterFree], 1);
  p.free_stack[idx] = page;
}
// drop one reference; the last owner returns the page to the free list
__device__ __forceinline__ void unref_page(const pace_kv_pool_t& p, int page) {
  if (page < 0 || page >= p.n_pages) return;
  if (atomicSub(&p.page_ref[page], 1) == 1) push_page(p, page);
}

__global__ void reset_kernel(pace_kv_pool_t p) {
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  const size_t nt = (size_t)p.max_seqs * p.max_pages_per_seq;
  for (size_t i = tid; i < nt; i += nth) p.block_table[i] = -1;
  for (size_t i = tid; i < (size_t)p.n_layers * p.max_seqs; i += nth) p.seq_len[i] = 0;
  for (size_t i = tid; i < (size_t)p.max_seqs; i += nth) p.seq_pages[i] = 0;
  for (size_t i = tid; i < (size_t)p.n_pages; i += nth) {
    p.page_ref[i] = 0;
    p.free_stack[i] = p.n_pages - 1 - (int)i;  // page 0 is handed out first
  }
  for (size_t i = tid; i < (size_t)(kCounterTicket + p.n_layers); i += nth) p.counters[i] = (i == kCounterFree) ? p.n_pages : 0;
  if (tid < 4) p.status[tid] = 0;
}

// One block.  Phase 1 (thread 0, sequential): copy-on-write of shared pages the
// coming append writes into.  Phase 2 (all threads): pop pages up to the needed
// count.  Phase 3 (all threads): copy the live rows of copied-on-write pages.
__global__ void reserve_kernel(pace_kv_pool_t p, int layer, const int32_t* __restrict__ seq_ids, int batch,
                               int n_new, const int32_t* __restrict__ n_per) {
  __shared__ int cow_count;
  int32_t* cow = p.table_tmp;  // triples (src page, dst page, rows)
  const int P = p.page_tokens;
  if (threadIdx.x == 0) {
    cow_count = 0;
    // pages are only ever shared after a beam gather; without one this sequential scan is skipped
    const int n_scan = p.counters[kCounterShared] ? batch : 0;
    for (int b = 0; b < n_scan; ++b) {
      const int slot = seq_ids[b];
      if (slot < 0 || slot >= p.max_seqs) continue;
      int n = n_per ? min(n_per[b], n_new) : n_new;
      if (n <= 0) continue;
      const int len = p.seq_len[(size_t)layer * p.max_seqs + slot];
      const int have = p.seq_pages[slot];
      const int need = min((len + n + P - 1) / P, p.max_pages_per_seq);
      int32_t* row = p.block_table + (size_t)slot * p.max_pages_per_seq;
      const int first = len / P;
      for (int lp = first; lp < min(have, need); ++lp) {
        const int pg = row[lp];
        if (pg < 0 || pg >= p.n_pages) continue;
        if (p.page_ref[pg] > 1) {
          const int np = pop_page(p);
          if (np < 0) {
            raise_status(p.status, PACE_DEV_POOL_EXHAUSTED);
            break;
          }
          p.page_ref[np] = 1;
          p.page_ref[pg] -= 1;
          row[lp] = np;
          const int rows = (lp == first) ? len - first * P : 0;
          if (rows > 0) {
            cow[3 * cow_count + 0] = pg;
            cow[3 * cow_count + 1] = np;
            cow[3 * cow_count + 2] = rows;
            ++cow_count;
          }
        }
      }
    }
  }
  __syncthreads();
  for (int b = threadIdx.x; b < batch; b += blockDim.x) {
    const int slot = seq_ids[b];
    if (slot < 0 || slot >= p.max_seqs) {
      raise_status(p.status, PACE_DEV_BAD_INDEX);
      continue;
    }
    int n = n_per ? min(n_per[b], n_new) : n_new;
    if (n <= 0) continue;
    const int len = p.seq_len[(size_t)layer * p.max_seqs + slot];
    int need = (len + n + P - 1) / P;
    if (need > p.max_pages_per_seq) {
      raise_status(p.status, PACE_DEV_TABLE_FULL);
      need = p.max_pages_per_seq;
    }
    int have = p.seq_pages[slot];
    int32_t* row = p.block_table + (size_t)slot * p.max_pages_per_seq;
    while (have < need) {
      const int np = pop_page(p);
      if (np < 0) {
        raise_status(p.status, PACE_DEV_POOL_EXHAUSTED);
        break;
      }
      p.page_ref[np] = 1;
      row[have++] = np;
    }
    p.seq_pages[slot] = have;
  }
  __syncthreads();
  const int nc = cow_count;
  if (nc == 0) return;
  // rows of a page are contiguous per head: copy rows*D elements for every (layer, K|V, head)
  const size_t page_elems = (size_t)p.n_kv_heads * P * p.head_dim;
  const size_t region = page_elems * (size_t)p.n_pages;
  uint4* base = reinterpret_cast<uint4*>(p.pages);
  const int vec_per_row = p.head_dim / 8;
  for (int c = 0; c < nc; ++c) {
    const int src = cow[3 * c], dst = cow[3 * c + 1], rows = cow[3 * c + 2];
    const size_t per_head = (size_t)rows * vec_per_row;
    const size_t total = (size_t)p.n_layers * 2 * p.n_kv_heads * per_head;
    for (size_t i = threadIdx.x; i < total; i += blockDim.x) {
      const size_t lk = i / (p.n_kv_heads * per_head);
      const size_t rem = i % (p.n_kv_heads * per_head);
      const size_t h = rem / per_head, o = rem % per_head;
      const size_t head_off = (h * P) * (size_t)p.head_dim / 8;
      const size_t s = (lk * region + (size_t)src * page_elems) / 8 + head_off + o;
      const size_t d = (lk * region + (size_t)dst * page_elems) / 8 + head_off + o;
      base[d] = base[s];
    }
  }
}

// The last block of an append grid to finish advances the per-layer lengths (a ticket counter in
// the pool tells which block that is, and is left at zero for the next launch).
__device__ __forceinline__ void advance_lengths_in_last_block(const pace_kv_pool_t& p, int layer,
                                                              const int32_t* __restrict__ seq_ids, int batch, int n_new,
                                                              const int32_t* __restrict__ n_per) {
  __shared__ int is_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int ticket = atomicAdd(&p.counters[kCounterTicket + layer], 1);
    is_last = (ticket == (int)gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    for (int b = threadIdx.x; b < batch; b += blockDim.x) {
      const int slot = seq_ids[b];
      if (slot < 0 || slot >= p.max_seqs) continue;
      const int n = n_per ? min(n_per[b], n_new) : n_new;
      if (n > 0) p.seq_len[(size_t)layer * p.max_seqs + slot] += n;
    }
    if (threadIdx.x == 0) p.counters[kCounterTicket + layer] = 0;
  }
}

// One warp per (sequence, new token, kv head): lanes [0, D/8) move the K row,
// lanes [16, 16 + D/8) the V row, 16 bytes per lane.  The last block to finish
// advances the per-layer lengths.
__global__ void __launch_bounds__(256)
    append_kernel(pace_kv_pool_t p, int layer, const int32_t* __restrict__ seq_ids, int batch, int n_new,
                  const int32_t* __restrict__ n_per, const __nv_bfloat16* __restrict__ k_new,
                  const __nv_bfloat16* __restrict__ v_new, int64_t sb, int64_t sh, int64_t st, int drain) {
  // the attention kernel behind this append may set up while the append runs
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // (The new rows are read with L2 loads, __ldcg: launched as a programmatic dependent this kernel does
  // not start with the cache maintenance of a kernel boundary behind it.)
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const long long total = (long long)batch * n_new * p.n_kv_heads;
  const int P = p.page_tokens, D = p.head_dim;
  const int vec_per_row = D / 8;
  const size_t page_elems = (size_t)p.n_kv_heads * P * D;
  const size_t region = page_elems * (size_t)p.n_pages;
  __nv_bfloat16* kbase = reinterpret_cast<__nv_bfloat16*>(p.pages) + ((size_t)layer * 2) * region;
  __nv_bfloat16* vbase = kbase + region;
  const int32_t* lens = p.seq_len + (size_t)layer * p.max_seqs;

  for (long long w = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); w < total;
       w += (long long)gridDim.x * warps_per_block) {
    const int h = (int)(w % p.n_kv_heads);
    const int t = (int)((w / p.n_kv_heads) % n_new);
    const int b = (int)(w / ((long long)p.n_kv_heads * n_new));
    const int slot = seq_ids[b];
    if (slot < 0 || slot >= p.max_seqs) continue;  // reported by reserve
    const int n = n_per ? min(n_per[b], n_new) : n_new;
    if (t >= n) continue;
    const int pos = lens[slot] + t;
    const int lp = pos / P;
    int page = -1;
    if (lp < p.max_pages_per_seq) page = p.block_table[(size_t)slot * p.max_pages_per_seq + lp];
    if (page < 0 || page >= p.n_pages) {
      if (lane == 0) raise_status(p.status, PACE_DEV_BAD_INDEX);
      continue;
    }
    const size_t dst = (((size_t)page * p.n_kv_heads + h) * P + (pos - lp * P)) * (size_t)D;
    const size_t src = (size_t)b * sb + (size_t)h * sh + (size_t)t * st;
    const int half = lane >> 4, l16 = lane & 15;
    if (l16 < vec_per_row) {
      const uint4* s = reinterpret_cast<const uint4*>((half ? v_new : k_new) + src) + l16;
      uint4* d = reinterpret_cast<uint4*>((half ? vbase : kbase) + dst) + l16;
      *d = __ldcg(s);
    }
  }
  advance_lengths_in_last_block(p, layer, seq_ids, batch, n_new, n_per);
  // Launched as a programmatic dependent, the append overlaps the attention kernel in front of it.
  // drain: it must not COMPLETE before that kernel does - the attention kernel behind the append
  // orders itself after the append only, and shares its workspace with the one in front.  The host
  // clears drain when the attention launch in front never touches the workspace: the launch behind
  // the append then learns of that launch's completion without the detour through this kernel's exit.
  if (drain) asm volatile("griddepcontrol.wait;" ::: "memory");
}

// The appends of a whole decode step in one launch: one warp per (layer, sequence).  The warp looks
// the sequence's slot, length and page up once, moves the rows of all KV heads (16 bytes per lane,
// the loads of up to eight rows in flight together) and then advances that one length itself - no
// other warp reads or writes it, so the launch needs neither a ticket nor a fence.  Meant for decode
// steps (a few tokens per sequence); a prefill chunk is better served by one append_kernel per layer.
// The kernel waits for everything in front of it on the stream before it touches anything (the
// step's attention launches read the lengths it advances), and nothing behind it starts early.
__global__ void __launch_bounds__(256)
    append_layers_kernel(pace_kv_pool_t p, int layer_begin, int layer_end, const int32_t* __restrict__ seq_ids, int batch,
                         int n_new, const int32_t* __restrict__ n_per, const __nv_bfloat16* __restrict__ k_new,
                         const __nv_bfloat16* __restrict__ v_new, int64_t sl, int64_t sb, int64_t sh, int64_t st) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int P = p.page_tokens, D = p.head_dim, H = p.n_kv_heads;
  const int vec_per_row = D / 8;             // 16-byte vectors in a row: 16 (D = 128) or 8
  const int rows_per_pass = 32 / vec_per_row;  // rows one pass of the warp moves: 2 or 4
  const size_t page_elems = (size_t)H * P * D;
  const size_t region = page_elems * (size_t)p.n_pages;
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= batch * (layer_end - layer_begin)) return;
  const int b = w % batch, li = w / batch, layer = layer_begin + li;
  const int slot = seq_ids[b];
  if (slot < 0 || slot >= p.max_seqs) return;  // reported by reserve
  const int n = n_per ? min(n_per[b], n_new) : n_new;
  if (n <= 0) return;
  int32_t* len_p = p.seq_len + (size_t)layer * p.max_seqs + slot;
  const int len = *len_p;
  __nv_bfloat16* kbase = reinterpret_cast<__nv_bfloat16*>(p.pages) + ((size_t)layer * 2) * region;
  const int r_in = lane / vec_per_row, vec = lane - r_in * vec_per_row;
  bool bad = false;
  for (int t = 0; t < n; ++t) {
    const int pos = len + t, lp = pos / P;
    int page = -1;
    if (lp < p.max_pages_per_seq) page = p.block_table[(size_t)slot * p.max_pages_per_seq + lp];
    if (page < 0 || page >= p.n_pages) {
      bad = true;
      continue;
    }
    // rows of this token: K of head 0 .. H-1, then V of head 0 .. H-1
    const size_t tok_src = (size_t)li * sl + (size_t)b * sb + (size_t)t * st;
    const size_t tok_dst = ((size_t)page * H * P + (pos - lp * P)) * (size_t)D;
    for (int r0 = 0; r0 < 2 * H; r0 += 4 * rows_per_pass) {
      uint4 val[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = r0 + u * rows_per_pass + r_in;
        if (r < 2 * H) {
          const int is_v = r >= H, h = is_v ? r - H : r;
          val[u] = __ldcg(reinterpret_cast<const uint4*>((is_v ? v_new : k_new) + tok_src + (size_t)h * sh) + vec);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = r0 + u * rows_per_pass + r_in;
        if (r < 2 * H) {
          const int is_v = r >= H, h = is_v ? r - H : r;
          reinterpret_cast<uint4*>(kbase + (is_v ? region : 0) + tok_dst + (size_t)h * P * D)[vec] = val[u];
        }
      }
    }
  }
  if (bad && lane == 0) raise_status(p.status, PACE_DEV_BAD_INDEX);
  __syncwarp();
  if (lane == 0) *len_p = len + n;
}

// The same step when its attention launches have already stored the rows (PACE_ATTN_PENDING_ROW):
// only the lengths are left to advance, one thread per (layer, sequence).
__global__ void advance_layers_kernel(pace_kv_pool_t p, int layer_begin, int layer_end, const int32_t* __restrict__ seq_ids,
                                      int batch, int n_new, const int32_t* __restrict__ n_per) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= batch * (layer_end - layer_begin)) return;
  const int b = i % batch, layer = layer_begin + i / batch;
  const int slot = seq_ids[b];
  if (slot < 0 || slot >= p.max_seqs) return;  // reported by reserve
  const int n = n_per ? min(n_per[b], n_new) : n_new;
  if (n > 0) p.seq_len[(size_t)layer * p.max_seqs + slot] += n;
}

// RoPE + append: eight lanes per (sequence, new token, group of kRopeHeads heads) of the projection
// outputs.  Query rows are rotated into q_out, key rows rotated into their cache slot, value rows
// copied into theirs.  A lane owns eight (x1, x2) pairs of every row of its group: it loads their
// fp32 cos and sin values once per token and then, per head, two 16-byte vectors in and two out.
// The arithmetic reproduces elementwise bf16 ops: cos and sin rounded to bf16 first, then every
// product and every sum rounded to bf16 (pace/ops/rotary_embedding.py:398-441).
struct RopeParams {
  const __nv_bfloat16 *q, *k, *v;
  __nv_bfloat16* q_out;
  int64_t q_sb, q_st, q_sh, k_sb, k_st, k_sh, v_sb, v_st, v_sh, o_sb, o_st, o_sh, row_sb;
  const int32_t* table_row;
  const float *cos_t, *sin_t;
  int table_rows, rotary_dim, gptj, n_q_heads;
  __nv_bfloat16 *k_stage, *v_stage;  // deferred append: K/V rows go here, not to the pool
  int64_t s_sb, s_sh, s_st;
};
constexpr int kRopeHeads = 6;  // heads per work item: 32 + 2 x 8 heads make eight items per token

__global__ void __launch_bounds__(256, 3)
    append_rope_kernel(pace_kv_pool_t p, int layer, const int32_t* __restrict__ seq_ids, int batch, int n_new,
                       const int32_t* __restrict__ n_per, RopeParams r, int drain) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int g = threadIdx.x & 7;
  const int P = p.page_tokens, D = p.head_dim, R = r.rotary_dim, Hkv = p.n_kv_heads, Hq = r.n_q_heads;
  const int heads = Hq + 2 * Hkv;
  const int groups = (heads + kRopeHeads - 1) / kRopeHeads;
  const long long total = (long long)batch * n_new * groups;
  const long long stride = (long long)gridDim.x * (blockDim.x >> 3);
  const size_t region = (size_t)Hkv * P * D * (size_t)p.n_pages;
  __nv_bfloat16* kbase = reinterpret_cast<__nv_bfloat16*>(p.pages) + ((size_t)layer * 2) * region;
  __nv_bfloat16* vbase = kbase + region;
  const int32_t* lens = p.seq_len + (size_t)layer * p.max_seqs;

  for (long long w = (long long)blockIdx.x * (blockDim.x >> 3) + (threadIdx.x >> 3); w < total; w += stride) {
    const int hg = (int)(w % groups);
    const int t = (int)((w / groups) % n_new);
    const int b = (int)(w / ((long long)groups * n_new));
    const int slot = seq_ids[b];
    if (slot < 0 || slot >= p.max_seqs) continue;  // reported by reserve
    const int n = n_per ? min(n_per[b], n_new) : n_new;
    if (t >= n) continue;
    // the token's cache row (key and value heads of this group go there)
    const bool staged = r.k_stage != nullptr;
    const int pos = staged ? 0 : lens[slot] + t;
    const int lp = pos / P;
    int page = -1;
    if (!staged && lp < p.max_pages_per_seq) page = p.block_table[(size_t)slot * p.max_pages_per_seq + lp];
    const bool page_ok = staged || (page >= 0 && page < p.n_pages);
    int row = r.table_row[(size_t)b * r.row_sb + t];
    if (row < 0 || row >= r.table_rows) {
      if (g == 0 && hg == 0) raise_status(p.status, PACE_DEV_BAD_INDEX);
      row = -1;  // the token passes through unrotated
    }
    // This lane's eight cos / sin values (rotation block g), rounded to bf16 and paired the way the
    // packed arithmetic below wants them: NeoX (c[2j], c[2j+1]), GPT-J (c[j], c[j]).  bf16x2
    // multiplies, adds and subtracts round every result to bf16 exactly like the elementwise ops.
    __nv_bfloat162 c2[8], s2[8];
    const bool turns = row >= 0 && g < R / 16;
    if (turns) {
      const float4* cp = reinterpret_cast<const float4*>(r.cos_t + (size_t)row * (R / 2) + 8 * g);
      const float4* sp = reinterpret_cast<const float4*>(r.sin_t + (size_t)row * (R / 2) + 8 * g);
      const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
      const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      if (r.gptj) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          c2[j] = __floats2bfloat162_rn(cs[j], cs[j]);
          s2[j] = __floats2bfloat162_rn(sn[j], sn[j]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          c2[j] = __floats2bfloat162_rn(cs[2 * j], cs[2 * j + 1]);
          s2[j] = __floats2bfloat162_rn(sn[2 * j], sn[2 * j + 1]);
        }
      }
    }
    const int offA = r.gptj ? 16 * g : 8 * g, offB = r.gptj ? 16 * g + 8 : R / 2 + 8 * g;

    const int h_end = min(heads, (hg + 1) * kRopeHeads);
    // the token's rows: everything but the head offset
    const __nv_bfloat16* const q_tok = r.q + (size_t)b * r.q_sb + (size_t)t * r.q_st;
    const __nv_bfloat16* const k_tok = r.k + (size_t)b * r.k_sb + (size_t)t * r.k_st;
    const __nv_bfloat16* const v_tok = r.v + (size_t)b * r.v_sb + (size_t)t * r.v_st;
    __nv_bfloat16* const o_tok = r.q_out + (size_t)b * r.o_sb + (size_t)t * r.o_st;
    const size_t cache_tok = ((size_t)page * Hkv * P + (pos - lp * P)) * (size_t)D;
    // Heads go three at a time: all loads of a batch are issued before its first store.  (q_out may be
    // q itself, so the compiler has to keep every load behind the stores in front of it; batching by
    // hand is what puts several rows in flight per lane.)
    constexpr int HB = 3;
    for (int h0 = hg * kRopeHeads; h0 < h_end; h0 += HB) {
      const __nv_bfloat16* src[HB];
      __nv_bfloat16* dst[HB];
      bool live[HB], is_v[HB];
      uint4 va[HB], vb[HB];
#pragma unroll
      for (int u = 0; u < HB; ++u) {
        const int hh = h0 + u;
        live[u] = hh < h_end;
        is_v[u] = hh >= Hq + Hkv;
        src[u] = nullptr;
        dst[u] = nullptr;
        if (!live[u]) continue;
        if (hh < Hq) {
          src[u] = q_tok + (size_t)hh * r.q_sh;
          dst[u] = o_tok + (size_t)hh * r.o_sh;
        } else {
          const int h = is_v[u] ? hh - Hq - Hkv : hh - Hq;
          src[u] = is_v[u] ? v_tok + (size_t)h * r.v_sh : k_tok + (size_t)h * r.k_sh;
          if (!page_ok) {
            if (g == 0) raise_status(p.status, PACE_DEV_BAD_INDEX);
            live[u] = false;
            continue;
          }
          dst[u] = staged ? (is_v[u] ? r.v_stage : r.k_stage) + (size_t)b * r.s_sb + (size_t)h * r.s_sh + (size_t)t * r.s_st
                          : (is_v[u] ? vbase : kbase) + cache_tok + (size_t)h * P * D;
        }
        if (turns && !is_v[u]) {
          va[u] = __ldcg(reinterpret_cast<const uint4*>(src[u] + offA));
          vb[u] = __ldcg(reinterpret_cast<const uint4*>(src[u] + offB));
        } else if (D == 128 || g < D / 16) {  // a row that is only copied: this lane's two vectors of it
          va[u] = __ldcg(reinterpret_cast<const uint4*>(src[u]) + g);
          vb[u] = __ldcg(reinterpret_cast<const uint4*>(src[u]) + g + D / 16);
        }
      }
#pragma unroll
      for (int u = 0; u < HB; ++u) {
        if (!live[u]) continue;
        const bool rotated = turns && !is_v[u];
        if (rotated) {
          __nv_bfloat162 xa[4], xb[4], oa[4], ob[4];
          *reinterpret_cast<uint4*>(xa) = va[u];
          *reinterpret_cast<uint4*>(xb) = vb[u];
          if (r.gptj) {
            // a register holds one pair (x1, x2): (x1 c, x2 c) + (-(x2 s), x1 s); the sign flip is exact
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const __nv_bfloat162 x = j < 4 ? xa[j] : xb[j - 4];
              const __nv_bfloat162 t = __hmul2_rn(x, c2[j]);
              __nv_bfloat162 w = __hmul2_rn(__lowhigh2highlow(x), s2[j]);   // (x2 s, x1 s)
              uint32_t bits = *reinterpret_cast<uint32_t*>(&w) ^ 0x00008000u;
              w = *reinterpret_cast<__nv_bfloat162*>(&bits);
              const __nv_bfloat162 o = __hadd2_rn(t, w);
              if (j < 4) oa[j] = o; else ob[j - 4] = o;
            }
          } else {
            // register j of the first half holds x1 of pairs 2j, 2j + 1, of the second half their x2
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              oa[j] = __hsub2_rn(__hmul2_rn(xa[j], c2[j]), __hmul2_rn(xb[j], s2[j]));
              ob[j] = __hadd2_rn(__hmul2_rn(xb[j], c2[j]), __hmul2_rn(xa[j], s2[j]));
            }
          }
          *reinterpret_cast<uint4*>(dst[u] + offA) = *reinterpret_cast<const uint4*>(oa);
          *reinterpret_cast<uint4*>(dst[u] + offB) = *reinterpret_cast<const uint4*>(ob);
          // elements beyond the rotated part
          for (int c = R / 8 + g; c < D / 8; c += 8)
            reinterpret_cast<uint4*>(dst[u])[c] = __ldcg(reinterpret_cast<const uint4*>(src[u]) + c);
        } else if (turns || row < 0 || is_v[u]) {
          const bool whole = is_v[u] || row < 0;  // value rows and unrotated tokens are copied whole
          if (whole) {
            if (D == 128 || g < D / 16) {
              reinterpret_cast<uint4*>(dst[u])[g] = va[u];
              reinterpret_cast<uint4*>(dst[u])[g + D / 16] = vb[u];
            }
          } else {
            for (int c = R / 8 + g; c < D / 8; c += 8)
              reinterpret_cast<uint4*>(dst[u])[c] = __ldcg(reinterpret_cast<const uint4*>(src[u]) + c);
          }
        } else {
          // a lane without a rotation block (rotary_dim < 128) of a rotated row: its share of the tail
          for (int c = R / 8 + g; c < D / 8; c += 8)
            reinterpret_cast<uint4*>(dst[u])[c] = __ldcg(reinterpret_cast<const uint4*>(src[u]) + c);
        }
      }
    }
  }
  if (r.k_stage == nullptr) advance_lengths_in_last_block(p, layer, seq_ids, batch, n_new, n_per);
  if (drain) asm volatile("griddepcontrol.wait;" ::: "memory");  // (see append_kernel)
}

__global__ void truncate_kernel(pace_kv_pool_t p, int layer_begin, int layer_end, const int32_t* __restrict__ seq_ids,
                                int batch, int remove_len, const int32_t* __restrict__ remove_per) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int n_l = layer_end - layer_begin;
  if (i >= batch * n_l) return;
  const int b = i % batch, layer = layer_begin + i / batch;
  const int slot = seq_ids[b];
  if (slot < 0 || slot >= p.max_seqs) {
    raise_status(p.status, PACE_DEV_BAD_INDEX);
    return;
  }
  const int r = remove_per ? remove_per[b] : remove_len;
  int32_t* len = p.seq_len + (size_t)layer * p.max_seqs + slot;
  if (r < 0 || r > *len) {
    raise_status(p.status, PACE_DEV_OVER_REMOVE);
    return;
  }
  *len -= r;
}

__global__ void release_kernel(pace_kv_pool_t p, const int32_t* __restrict__ seq_ids, int batch) {
  for (int b = blockIdx.x; b < batch; b += gridDim.x) {
    const int slot = seq_ids[b];
    if (slot < 0 || slot >= p.max_seqs) {
      if (threadIdx.x == 0) raise_status(p.status, PACE_DEV_BAD_INDEX);
      continue;
    }
    int32_t* row = p.block_table + (size_t)slot * p.max_pages_per_seq;
    const int have = p.seq_pages[slot];
    for (int lp = threadIdx.x; lp < have; lp += blockDim.x) {
      unref_page(p, row[lp]);
      row[lp] = -1;
    }
    for (int l = threadIdx.x; l < p.n_layers; l += blockDim.x) p.seq_len[(size_t)l * p.max_seqs + slot] = 0;
    __syncthreads();
    if (threadIdx.x == 0) p.seq_pages[slot] = 0;
    __syncthreads();
  }
}

// One block.  Row i of the batch becomes old row beam_idx[i]: snapshot the source
// rows, take references on them, drop the references of the rows being replaced,
// then write the snapshot back.
__global__ void gather_kernel(pace_kv_pool_t p, const int32_t* __restrict__ seq_ids,
                              const int64_t* __restrict__ beam_idx, int batch) {
  const int MP = p.max_pages_per_seq;
  int32_t* tmp_rows = p.table_tmp;                         // [batch][MP + 1] (last = page count)
  int32_t* tmp_len = p.table_tmp + (size_t)p.max_seqs * (MP + 4);  // [n_layers][batch]
  __shared__ int bad;
  if (threadIdx.x == 0) {
    bad = 0;
    p.counters[kCounterShared] = 1;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < batch; i += blockDim.x) {
    const long long j = beam_idx[i];
    const int dst = seq_ids[i];
    if (j < 0 || j >= batch || dst < 0 || dst >= p.max_seqs) bad = 1;
    else {
      const int src = seq_ids[j];
      if (src < 0 || src >= p.max_seqs) bad = 1;
    }
  }
  __syncthreads();
  if (bad) {
    if (threadIdx.x == 0) raise_status(p.status, PACE_DEV_BAD_INDEX);
    return;
  }
  for (int i = 0; i < batch; ++i) {
    const int src = seq_ids[beam_idx[i]];
    const int have = p.seq_pages[src];
    for (int lp = threadIdx.x; lp < MP; lp += blockDim.x)
      tmp_rows[(size_t)i * (MP + 1) + lp] = lp < have ? p.block_table[(size_t)src * MP + lp] : -1;
    if (threadIdx.x == 0) tmp_rows[(size_t)i * (MP + 1) + MP] = have;
    for (int l = threadIdx.x; l < p.n_layers; l += blockDim.x)
      tmp_len[(size_t)l * batch + i] = p.seq_len[(size_t)l * p.max_seqs + src];
  }
  __syncthreads();
  for (int i = 0; i < batch; ++i) {
    const int have = tmp_rows[(size_t)i * (MP + 1) + MP];
    for (int lp = threadIdx.x; lp < have; lp += blockDim.x) {
      const int pg = tmp_rows[(size_t)i * (MP + 1) + lp];
      if (pg >= 0 && pg < p.n_pages) atomicAdd(&p.page_ref[pg], 1);
    }
  }
  __syncthreads();
  for (int i = 0; i < batch; ++i) {
    const int dst = seq_ids[i];
    const int have = p.seq_pages[dst];
    for (int lp = threadIdx.x; lp < have; lp += blockDim.x) unref_page(p, p.block_table[(size_t)dst * MP + lp]);
  }
  __syncthreads();
  for (int i = 0; i < batch; ++i) {
    const int dst = seq_ids[i];
    for (int lp = threadIdx.x; lp < MP; lp += blockDim.x)
      p.block_table[(size_t)dst * MP + lp] = tmp_rows[(size_t)i * (MP + 1) + lp];
    if (threadIdx.x == 0) p.seq_pages[dst] = tmp_rows[(size_t)i * (MP + 1) + MP];
    for (int l = threadIdx.x; l < p.n_layers; l += blockDim.x)
      p.seq_len[(size_t)l * p.max_seqs + dst] = tmp_len[(size_t)l * batch + i];
  }
}

// PARD acceptance, one thread per sequence (a handful of integer comparisons each).
__global__ void pard_accept_kernel(const int64_t* __restrict__ drafts, const int64_t* __restrict__ target_next,
                                   const int32_t* __restrict__ n_target, const uint8_t* __restrict__ forced, int batch, int d,
                                   int32_t* __restrict__ keep_out, int32_t* __restrict__ target_remove,
                                   int32_t* __restrict__ draft_remove, int64_t* __restrict__ kept) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const int64_t* dr = drafts + (size_t)b * d;
  const int64_t* tn = target_next + (size_t)b * (d + 1);
  const int nt = max(1, min(n_target[b], d + 1));
  int keep = 0;
  for (int i = 0; i < d - 1; ++i) {
    const bool ok = forced ? forced[(size_t)b * (d - 1) + i] != 0 : (i < nt && tn[i] == dr[i]);
    if (!ok) break;
    ++keep;
  }
  ++keep;  // the target's own token is always kept
  for (int i = 0; i < keep - 1; ++i) kept[(size_t)b * d + i] = forced ? dr[i] : tn[i];
  kept[(size_t)b * d + keep - 1] = tn[min(keep - 1, nt - 1)];
  keep_out[b] = keep;
  target_remove[b] = d - keep > 0 ? d - keep + 1 : 0;
  draft_remove[b] = d - 1;
}

// Dense read-back: one 16-byte vector per thread.
__global__ void read_dense_kernel(pace_kv_pool_t p, int layer, const int32_t* __restrict__ seq_ids, int batch,
                                  uint4* __restrict__ k_out, uint4* __restrict__ v_out, int cap) {
  const int P = p.page_tokens, D = p.head_dim, H = p.n_kv_heads;
  const int vpr = D / 8;
  const size_t total = (size_t)batch * H * cap * vpr;
  const size_t page_elems = (size_t)H * P * D;
  const size_t region = page_elems * (size_t)p.n_pages;
  const uint4* kbase = reinterpret_cast<const uint4*>(reinterpret_cast<__nv_bfloat16*>(p.pages) +
                                                      ((size_t)layer * 2) * region);
  const uint4* vbase = kbase + region / 8;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % vpr);
    const int t = (int)((i / vpr) % cap);
    const int h = (int)((i / ((size_t)vpr * cap)) % H);
    const int b = (int)(i / ((size_t)vpr * cap * H));
    uint4 kv = make_uint4(0, 0, 0, 0), vv = kv;
    const int slot = seq_ids[b];
    if (slot >= 0 && slot < p.max_seqs) {
      const int lp = t / P;
      if (lp < p.seq_pages[slot] && lp < p.max_pages_per_seq) {
        const int pg = p.block_table[(size_t)slot * p.max_pages_per_seq + lp];
        if (pg >= 0 && pg < p.n_pages) {
          const size_t off = ((((size_t)pg * H + h) * P + (t - lp * P)) * D) / 8 + c;
          kv = kbase[off];
          vv = vbase[off];
        }
      }
    }
    k_out[i] = kv;
    v_out[i] = vv;
  }
}

// Whether an append to `layer` of this pool may be launched as a programmatic dependent, i.e. start
// while this library's newest attention launch on the stream is still running.  Not when that
// launch reads the same layer of the same pool (its blocks may still be reading the lengths the
// append advances), and not when the append rewrites the buffer that launch takes its queries from.
bool append_may_overlap(cudaStream_t stream, const pace_kv_pool_t* p, int layer, const void* rewritten = nullptr) {
  const StreamNote n = stream_note(stream);
  if (n.pages == p->pages && (n.layer == layer || p->n_layers == 1)) return false;
  if (rewritten && n.q == rewritten) return false;
  return true;
}

bool pool_ok(const pace_kv_pool_t* p) {
  return geometry_ok(p) && p->pages && p->block_table && p->seq_len && p->seq_pages && p->page_ref &&
         p->free_stack && p->counters && p->status && p->table_tmp;
}

}  // namespace
}  // namespace pace

using namespace pace;

extern "C" {

const char* pace_last_cuda_error(void) { return g_err; }
const char* pace_version(void) { return "pace_b200 0.1 (sm_100a)"; }

int pace_kv_pool_bytes(const pace_kv_pool_t* g, uint64_t* pages_bytes, uint64_t* meta_bytes) {
  if (!geometry_ok(g) || !pages_bytes || !meta_bytes) return PACE_ERR_INVALID;
  *pages_bytes = (uint64_t)g->n_layers * 2 * g->n_pages * g->n_kv_heads * g->page_tokens * g->head_dim * 2;
  *meta_bytes = meta_layout(g).total;
  return PACE_OK;
}

int pace_kv_pool_bind(pace_kv_pool_t* p, void* pages_mem, void* meta_mem) {
  if (!geometry_ok(p) || !pages_mem || !meta_mem) return PACE_ERR_INVALID;
  if (((uintptr_t)pages_mem & 255) || ((uintptr_t)meta_mem & 255)) return PACE_ERR_INVALID;
  const MetaLayout m = meta_layout(p);
  char* b = static_cast<char*>(meta_mem);
  p->pages = pages_mem;
  p->block_table = reinterpret_cast<int32_t*>(b + m.block_table);
  p->seq_len = reinterpret_cast<int32_t*>(b + m.seq_len);
  p->seq_pages = reinterpret_cast<int32_t*>(b + m.seq_pages);
  p->page_ref = reinterpret_cast<int32_t*>(b + m.page_ref);
  p->free_stack = reinterpret_cast<int32_t*>(b + m.free_stack);
  p->counters = reinterpret_cast<int32_t*>(b + m.counters);
  p->status = reinterpret_cast<int32_t*>(b + m.status);
  p->table_tmp = reinterpret_cast<int32_t*>(b + m.table_tmp);
  p->owns_memory = 0;
  return PACE_OK;
}

int pace_kv_pool_create(pace_kv_pool_t* p) {
  uint64_t pb = 0, mb = 0;
  if (pace_kv_pool_bytes(p, &pb, &mb) != PACE_OK) return PACE_ERR_INVALID;
  void *pages = nullptr, *meta = nullptr;
  PACE_CUDA_TRY(cudaMalloc(&pages, pb));
  cudaError_t e = cudaMalloc(&meta, mb);
  if (e != cudaSuccess) {
    cudaFree(pages);
    set_cuda_error(e, "cudaMalloc(meta)");
    return PACE_ERR_CUDA;
  }
  pace_kv_pool_bind(p, pages, meta);
  p->owns_memory = 1;
  return pace_kv_pool_reset(p, nullptr);
}

int pace_kv_pool_destroy(pace_kv_pool_t* p) {
  if (!p) return PACE_ERR_INVALID;
  if (p->owns_memory) {
    PACE_CUDA_TRY(cudaFree(p->pages));
    PACE_CUDA_TRY(cudaFree(p->block_table));  // first array of the meta block
  }
  p->pages = nullptr;
  p->block_table = p->seq_len = p->seq_pages = p->page_ref = p->free_stack = nullptr;
  p->counters = p->status = p->table_tmp = nullptr;
  p->owns_memory = 0;
  return PACE_OK;
}

int pace_kv_pool_reset(const pace_kv_pool_t* p, void* stream) {
  if (!pool_ok(p)) return PACE_ERR_INVALID;
  reset_kernel<<<148, 256, 0, (cudaStream_t)stream>>>(*p);
  PACE_LAUNCH_CHECK("reset_kernel");
  note_pool_write((cudaStream_t)stream);
  return PACE_OK;
}

int pace_kv_pool_query(const pace_kv_pool_t* p, int32_t out[4], void* stream) {
  if (!pool_ok(p) || !out) return PACE_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  int32_t st = 0, fr = 0;
  PACE_CUDA_TRY(cudaMemcpyAsync(&st, p->status, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  PACE_CUDA_TRY(cudaMemcpyAsync(&fr, p->counters, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  PACE_CUDA_TRY(cudaStreamSynchronize(s));
  out[0] = st;
  out[1] = fr;
  out[2] = out[3] = 0;
  return PACE_OK;
}

int pace_kv_pool_clear_status(const pace_kv_pool_t* p, void* stream) {
  if (!pool_ok(p)) return PACE_ERR_INVALID;
  PACE_CUDA_TRY(cudaMemsetAsync(p->status, 0, 4 * sizeof(int32_t), (cudaStream_t)stream));
  return PACE_OK;
}

int pace_kv_seq_release(const pace_kv_pool_t* p, const int32_t* seq_ids, int32_t batch, void* stream) {
  if (!pool_ok(p) || !seq_ids || batch < 0) return PACE_ERR_INVALID;
  if (batch == 0) return PACE_OK;
  release_kernel<<<batch < 148 ? batch : 148, 128, 0, (cudaStream_t)stream>>>(*p, seq_ids, batch);
  PACE_LAUNCH_CHECK("release_kernel");
  note_pool_write((cudaStream_t)stream);
  return PACE_OK;
}

int pace_kv_reserve(const pace_kv_pool_t* p, int32_t layer, const int32_t* seq_ids, int32_t batch, int32_t n_new,
                    const int32_t* n_per, void* stream) {
  if (!pool_ok(p) || !seq_ids || batch < 0 || batch > p->max_seqs || n_new < 0 || layer < 0 ||
      layer >= p->n_layers)
    return PACE_ERR_INVALID;
  if (batch == 0 || n_new == 0) return PACE_OK;
  reserve_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(*p, layer, seq_ids, batch, n_new, n_per);
  PACE_LAUNCH_CHECK("reserve_kernel");
  note_pool_write((cudaStream_t)stream);
  return PACE_OK;
}

int pace_kv_append(const pace_kv_pool_t* p, int32_t layer, const int32_t* seq_ids, int32_t batch, int32_t n_new,
                   const int32_t* n_per, const void* k_new, const void* v_new, int64_t sb, int64_t sh, int64_t st,
                   void* stream) {
  if (!pool_ok(p) || !seq_ids || batch < 0 || batch > p->max_seqs || n_new < 0 || layer < 0 ||
      layer >= p->n_layers)
    return PACE_ERR_INVALID;
  if (batch == 0 || n_new == 0) return PACE_OK;
  if (!k_new || !v_new) return PACE_ERR_INVALID;
  PACE_PROFILE("kv_append", stream, "layer=%d batch=%d n_new=%d", layer, batch, n_new);
  // 16-byte vector moves: bases and strides must keep rows 16-byte aligned
  if (((uintptr_t)k_new & 15) || ((uintptr_t)v_new & 15) || (sb & 7) || (sh & 7) || (st & 7)) return PACE_ERR_INVALID;
  const long long warps = (long long)batch * n_new * p->n_kv_heads;
  long long blocks = (warps + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  // Programmatic dependent launch: when the kernel in front of this one on the stream announces it
  // (the attention kernels do, and an append touches nothing they read or write - another layer's
  // pages and lengths), the append overlaps with it instead of waiting for it to drain.  After any
  // other kernel the attribute changes nothing.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = append_may_overlap((cudaStream_t)stream, p, layer) ? 1 : 0;
  PACE_CUDA_TRY(cudaLaunchKernelEx(&cfg, append_kernel, *p, (int)layer, seq_ids, (int)batch, (int)n_new, n_per,
                                   (const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, (int64_t)sb, (int64_t)sh,
                                   (int64_t)st, front_attention_uses_workspace((cudaStream_t)stream) ? 1 : 0));
  PACE_LAUNCH_CHECK("append_kernel");
  note_pool_write((cudaStream_t)stream);
  return PACE_OK;
}

int pace_kv_append_layers(const pace_kv_pool_t* p, int32_t layer_begin, int32_t layer_end, const int32_t* seq_ids,
                          int32_t batch, int32_t n_new, const int32_t* n_per, const void* k_new, const void* v_new,
                          int64_t sl, int64_t sb, int64_t sh, int64_t st, void* stream) {
  if (!pool_ok(p) || !seq_ids || batch < 0 || batch > p->max_seqs || n_new < 0 || layer_begin < 0 ||
      layer_end > p->n_layers || layer_begin > layer_end)
    return PACE_ERR_INVALID;
  if (batch == 0 || n_new == 0 || layer_begin == layer_end) return PACE_OK;
  const bool lengths_only = !k_new && !v_new;  // the rows are in the pool already
  PACE_PROFILE("kv_append_layers", stream, "layers=%d..%d batch=%d n_new=%d rows=%d", layer_begin, layer_end, batch, n_new,
               lengths_only ? 0 : 1);
  if (!lengths_only && (!k_new || !v_new)) return PACE_ERR_INVALID;
  if (!lengths_only &&
      (((uintptr_t)k_new & 15) || ((uintptr_t)v_new & 15) || (sl & 7) || (sb & 7) || (sh & 7) || (st & 7)))
    return PACE_ERR_INVALID;
  const long long warps = (long long)batch * (layer_end - layer_begin);
  if (warps > (1LL << 30)) return PACE_ERR_UNSUPPORTED;
  // Launched as a programmatic dependent so that the launch itself overlaps the tail of the kernel in
  // front; the kernel's first instruction waits for that kernel (and everything older) to complete.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((warps + 7) / 8));
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (lengths_only) {
    cfg.gridDim = dim3((unsigned)((warps + 255) / 256));
    PACE_CUDA_TRY(cudaLaunchKernelEx(&cfg, advance_layers_kernel, *p, (int)layer_begin, (int)layer_end, seq_ids, (int)batch,
                                     (int)n_new, n_per));
    PACE_LAUNCH_CHECK("advance_layers_kernel");
    note_pool_write((cudaStream_t)stream);
    return PACE_OK;
  }
  PACE_CUDA_TRY(cudaLaunchKernelEx(&cfg, append_layers_kernel, *p, (int)layer_begin, (int)layer_end, seq_ids, (int)batch,
                                   (int)n_new, n_per, (const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new,
                                   (int64_t)sl, (int64_t)sb, (int64_t)sh, (int64_t)st));
  PACE_LAUNCH_CHECK("append_layers_kernel");
  note_pool_write((cudaStream_t)stream);
  return PACE_OK;
}

int pace_kv_append_rope(const pace_kv_pool_t* p, int32_t layer, const int32_t* seq_ids, int32_t batch, int32_t n_new,
                        const int32_t* n_per, const pace_rope_args_t* a, void* stream) {
  if (!pool_ok(p) || !seq_ids || !a || batch < 0 || batch > p->max_seqs || n_new < 0 || layer < 0 ||
      layer >= p->n_layers)
    return PACE_ERR_INVALID;
  if (batch == 0 || n_new == 0) return PACE_OK;
  if (!a->q || !a->k || !a->v || !a->q_out || !a->table_row || !a->cos_table || !a->sin_table) return PACE_ERR_INVALID;
  PACE_PROFILE("kv_append_rope", stream, "layer=%d batch=%d n_new=%d", layer, batch, n_new);
  if (a->n_q_heads < 1 || a->table_rows < 1 || a->rotary_dim < 16 || a->rotary_dim > p->head_dim || (a->rotary_dim & 15))
    return PACE_ERR_INVALID;
  // 16-byte vector moves: bases and strides must keep rows 16-byte aligned
  const uintptr_t bases = (uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->q_out |
                          (uintptr_t)a->cos_table | (uintptr_t)a->sin_table;
  const int64_t strides = a->q_stride_b | a->q_stride_t | a->q_stride_h | a->k_stride_b | a->k_stride_t | a->k_stride_h |
                          a->v_stride_b | a->v_stride_t | a->v_stride_h | a->o_stride_b | a->o_stride_t | a->o_stride_h;
  if ((bases & 15) || (strides & 7)) return PACE_ERR_INVALID;
  RopeParams r;
  r.q = (const __nv_bfloat16*)a->q;
  r.k = (const __nv_bfloat16*)a->k;
  r.v = (const __nv_bfloat16*)a->v;
  r.q_out = (__nv_bfloat16*)a->q_out;
  r.q_sb = a->q_stride_b; r.q_st = a->q_stride_t; r.q_sh = a->q_stride_h;
  r.k_sb = a->k_stride_b; r.k_st = a->k_stride_t; r.k_sh = a->k_stride_h;
  r.v_sb = a->v_stride_b; r.v_st = a->v_stride_t; r.v_sh = a->v_stride_h;
  r.o_sb = a->o_stride_b; r.o_st = a->o_stride_t; r.o_sh = a->o_stride_h;
  r.row_sb = a->row_stride_b;
  r.table_row = a->table_row;
  r.cos_t = a->cos_table;
  r.sin_t = a->sin_table;
  r.table_rows = a->table_rows;
  r.rotary_dim = a->rotary_dim;
  r.gptj = a->gptj_pairs ? 1 : 0;
  r.n_q_heads = a->n_q_heads;
  r.k_stage = (__nv_bfloat16*)a->k_stage;
  r.v_stage = (__nv_bfloat16*)a->v_stage;
  r.s_sb = a->stage_stride_b; r.s_sh = a->stage_stride_h; r.s_st = a->stage_stride_t;
  if (a->k_stage) {
    if (!a->v_stage || (((uintptr_t)a->k_stage | (uintptr_t)a->v_stage) & 15) ||
        ((a->stage_stride_b | a->stage_stride_h | a->stage_stride_t) & 7))
      return PACE_ERR_INVALID;
  }
  if (a->rotary_dim > 128) return PACE_ERR_UNSUPPORTED;  // eight lanes x 16 elements cover a row's rotated part
  const int groups = (a->n_q_heads + 2 * p->n_kv_heads + kRopeHeads - 1) / kRopeHeads;
  const long long items = (long long)batch * n_new * groups;
  long long blocks = (items + 31) / 32;  // 32 eight-lane groups per block
  if (blocks > 148 * 8) blocks = 148 * 8;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = append_may_overlap((cudaStream_t)stream, p, layer, a->q_out) ? 1 : 0;
  PACE_CUDA_TRY(cudaLaunchKernelEx(&cfg, append_rope_kernel, *p, (int)layer, seq_ids, (int)batch, (int)n_new, n_per, r,
                                   front_attention_uses_workspace((cudaStream_t)stream) ? 1 : 0));
  PACE_LAUNCH_CHECK("append_rope_kernel");
  if (!a->k_stage) note_pool_write((cudaStream_t)stream);  // (staged rows leave the pool as it was)
  return PACE_OK;
}

int pace_kv_truncate(const pace_kv_pool_t* p, int32_t layer_begin, int32_t layer_end, const int32_t* seq_ids,
                     int32_t batch, int32_t remove_len, const int32_t* remove_per, void* stream) {
  if (!pool_ok(p) || !seq_ids || batch < 0 || layer_begin < 0 || layer_end > p->n_layers ||
      layer_begin > layer_end || (!remove_per && remove_len < 0))
    return PACE_ERR_INVALID;
  const int n = batch * (layer_end - layer_begin);
  if (n == 0) return PACE_OK;
  PACE_PROFILE("kv_truncate", stream, "layers=%d..%d batch=%d", layer_begin, layer_end, batch);
  truncate_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(*p, layer_begin, layer_end, seq_ids, batch,
                                                                    remove_len, remove_per);
  PACE_LAUNCH_CHECK("truncate_kernel");
  note_pool_write((cudaStream_t)stream);
  return PACE_OK;
}

int pace_pard_accept(const int64_t* drafts, const int64_t* target_next, const int32_t* n_target, const uint8_t* forced,
                     int32_t batch, int32_t d, int32_t* keep, int32_t* target_remove, int32_t* draft_remove, int64_t* kept,
                     void* stream) {
  if (!drafts || !target_next || !n_target || !keep || !target_remove || !draft_remove || !kept || batch < 0 || d < 1)
    return PACE_ERR_INVALID;
  if (batch == 0) return PACE_OK;
  pard_accept_kernel<<<(batch + 127) / 128, 128, 0, (cudaStream_t)stream>>>(drafts, target_next, n_target, forced, batch, d,
                                                                           keep, target_remove, draft_remove, kept);
  PACE_LAUNCH_CHECK("pard_accept_kernel");
  return PACE_OK;
}

int pace_kv_gather(const pace_kv_pool_t* p, const int32_t* seq_ids, const int64_t* beam_idx, int32_t batch,
                   void* stream) {
  if (!pool_ok(p) || !seq_ids || !beam_idx || batch < 0 || batch > p->max_seqs) return PACE_ERR_INVALID;
  if (batch == 0) return PACE_OK;
  PACE_PROFILE("kv_gather", stream, "batch=%d", batch);
  gather_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(*p, seq_ids, beam_idx, batch);
  PACE_LAUNCH_CHECK("gather_kernel");
  note_pool_write((cudaStream_t)stream);
  return PACE_OK;
}

int pace_kv_read_dense(const pace_kv_pool_t* p, int32_t layer, const int32_t* seq_ids, int32_t batch, void* k_out,
                       void* v_out, int32_t cap, void* stream) {
  if (!pool_ok(p) || !seq_ids || batch < 0 || cap < 0 || layer < 0 || layer >= p->n_layers) return PACE_ERR_INVALID;
  if (batch == 0 || cap == 0) return PACE_OK;
  if (!k_out || !v_out || ((uintptr_t)k_out & 15) || ((uintptr_t)v_out & 15)) return PACE_ERR_INVALID;
  const size_t total = (size_t)batch * p->n_kv_heads * cap * (p->head_dim / 8);
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  read_dense_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(*p, layer, seq_ids, batch, (uint4*)k_out,
                                                                  (uint4*)v_out, cap);
  PACE_LAUNCH_CHECK("read_dense_kernel");
  return PACE_OK;
}

}  // extern "C"
