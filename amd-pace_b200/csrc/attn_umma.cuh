// 5th-generation tensor-core path of the multi-token attention kernel (prefill chunks, PARD verify).
//
// S = Q K^T and O += P V are tcgen05.mma instructions issued by one elected thread of an issuer warp,
// K and V in shared memory (K-major / MN-major, 128-byte swizzle, exactly the layout the tiled TMA
// copies produce), accumulators in tensor memory.  Two softmax warpgroups, A and B, each with its own
// running (max, sum), score / probability buffers and O accumulator, so that they never wait for one
// another while a unit part streams.  Two forms:
//   narrow  one 128-row query tile per unit; the chunks of a CTA's range are dealt alternately to the
//           groups (A: even, B: odd) and the two accumulators are merged when the part ends;
//   wide    256 query rows per unit = two 128-row tiles that share every K/V chunk the CTA fetches
//           (half the L2 -> SM traffic per flop); group A owns tile A, group B tile B, both work on
//           every chunk, nothing is merged inside the CTA.
// Tensor memory:
//     columns [0, 64) / [64, 128)    S_A / S_B: the scores of the chunk a group works on, 128 x 64 fp32
//     columns [128, 160) / [160, 192) P_A / P_B: its probabilities, 128 x 64 bf16 (two per column)
//     columns [192, 256)             a Q tile, 128 x D bf16 (two elements per column)
//     columns [256, 384) / [384, 512) O_A / O_B, 128 x D fp32
// A softmax thread owns one query row (TMEM lane == row): tcgen05.ld the row of S - which hands the
// score buffer back at once, so the QK of the group's next chunk runs while this one's softmax does -
// online softmax in registers, P stored to the group's P buffer as packed bf16 pairs once the PV of its
// previous chunk has completed; the second MMA takes it from there as its A operand.  Q sits in tensor
// memory as well (each softmax thread stores its own row once per unit part) and is the A operand of the
// first MMA: with Q in shared memory every chunk re-read the whole 32 KB tile, a third of the SM's
// shared-memory traffic, and shared-memory bandwidth paced those MMAs.  (The wide form's second tile
// does keep its Q in shared memory: tensor memory has room for one.)  O is rescaled in TMEM only when a
// row's running maximum grows by more than 2^8 (the result is exact either way: numerator and
// denominator share whatever maximum was used).
//
// Included by attn_mma.cu, which provides MmaParams, MetaM, the ring and its producer warp.
#pragma once

namespace pace {
namespace {

constexpr int kUmmaRows = 128;          // query rows per tile (UMMA M)
constexpr int kUmmaSoftmaxThreads = 256;  // two warpgroups
// Warps 0-7: softmax; 8: producer; 9: QK issuer (of group A's chunks when the work is split); 10: PV issuer;
// 11: narrow form: QK issuer of group B's chunks; wide form: PV issuer of group B.  (Issuers on warps 10 and 11, away from
// the schedulers of the softmax warps that hold a verify tile's live rows, measured the same.)
constexpr int kUmmaQkWarp = 9, kUmmaPvWarp = 10, kUmmaWarpB = 11;
constexpr int kTmemCols = 512;          // the whole tensor memory of the SM:
constexpr uint32_t kTmemO = 256;        //   [0, 128) S_A S_B, [128, 192) P_A P_B, [192, 256) Q, [256, 512) O_A O_B
constexpr uint32_t kTmemP = 128, kTmemQ = 192;
constexpr float kLazyRescale = 8.0f;    // log2 units
// Wide form: every n-th pair of a row's scores takes 2^x on the FMA pipe (0: none).  Both groups are in
// their exp2 phase at the same time there (they wait for the same K/V chunk) and the one exp2 unit per
// scheduler serves two warps: 1150 cycles per chunk for 2 x 64 exp2 per lane, measured.
constexpr int kWidePolyEvery = 2;
constexpr unsigned kSoftmaxBackoffNs = 100;  // a waiting softmax warp leaves its scheduler's issue slots to the MMA issuer

struct UmmaCtx {
  unsigned char* ring;    // [n_stages][K | V] as the TMA boxes land
  const MetaM* metas;
  uint64_t* full_bar;
  uint64_t* empty_bar;
  uint64_t* s_full;       // [2] per group: QK^T of its chunk has landed in TMEM
  uint64_t* s_free;       // [2] per group: every row of S is in registers (one arrival per warp of the group)
  uint64_t* p_full;       // [2] per group: P is in place (and O has been rescaled); one arrival per warp of the group
  uint64_t* o_full;       // [2] per group: PV of a chunk has been accumulated (and has read P)
  uint64_t* q_ready;      // the Q tile of a unit part is in tensor memory (one arrival per softmax warp)
  uint64_t* drain;        // [2] every MMA an issuer warp issued has completed
  uint64_t* drain_b;      // the same for warp 11 (second QK issuer or second PV issuer)
  unsigned char* qsw;     // wide form: tile B's Q, K-major 128-byte-swizzled: [D/64][128 rows][128 B]
  uint64_t* pub;          // meeting point of the 256 softmax threads while a cut unit is published
  uint64_t* xch;          // the two groups have posted their (max, sum) of a part (one arrival per warp)
  uint32_t* tmem_slot;    // where tcgen05.alloc wrote the base address
  int* flag;              // "this CTA arrived last" broadcast
  volatile int* abort;
  int n_my, n_stages, cta;
};

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
  const uint32_t hi = ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
  return ((uint64_t)hi << 32) | lo;
}
// instruction descriptor: bf16 x bf16 -> fp32, M = 128, A K-major
__host__ __device__ constexpr uint32_t umma_idesc(int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(kUmmaRows >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// A operand in tensor memory (128 lanes x 8 columns of packed bf16 pairs per 16-wide k-step)
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// Blackwell's two-wide fp32 arithmetic and three-input maximum: a row of 64 scores takes 32 instructions
// for the maximum, 32 for scale-and-shift and 32 for the row sum instead of 64 each - the softmax
// warps share their schedulers' issue slots with each other and the exp2 unit is the pipe to keep busy.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// 2^x for two values at once on the FMA pipe (any x; below -126 the result is 2^-126): round to the
// nearest integer with the 1.5 * 2^23 trick, a degree-3 polynomial for 2^f on [-0.5, 0.5] (relative error
// 1e-4, a twentieth of the bf16 rounding of P) and the integer part added into the exponent field.
__device__ __forceinline__ void exp2_poly2(float x0, float x1, float& p0, float& p1) {
  const uint32_t kMagic = 0x4B400000u, kNegMagic = 0xCB400000u, kNegOne = 0xBF800000u;  // 1.5 * 2^23, -1.5 * 2^23, -1.0
  x0 = fmaxf(x0, -126.f);
  x1 = fmaxf(x1, -126.f);
  uint64_t x, r, f, q;
  asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "r"(__float_as_uint(x0)), "r"(__float_as_uint(x1)));
  uint64_t magic, neg_magic, neg_one, c0, c1, c2, c3;
  asm("mov.b64 %0, {%1, %1};" : "=l"(magic) : "r"(kMagic));
  asm("mov.b64 %0, {%1, %1};" : "=l"(neg_magic) : "r"(kNegMagic));
  asm("mov.b64 %0, {%1, %1};" : "=l"(neg_one) : "r"(kNegOne));
  asm("mov.b64 %0, {%1, %1};" : "=l"(c0) : "r"(__float_as_uint(0.9999281764f)));
  asm("mov.b64 %0, {%1, %1};" : "=l"(c1) : "r"(__float_as_uint(0.6932609677f)));
  asm("mov.b64 %0, {%1, %1};" : "=l"(c2) : "r"(__float_as_uint(0.2426091731f)));
  asm("mov.b64 %0, {%1, %1};" : "=l"(c3) : "r"(__float_as_uint(0.05517086014f)));
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(x), "l"(magic));  // low mantissa bits: the rounded integer
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(f) : "l"(r), "l"(neg_magic));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(f) : "l"(f), "l"(neg_one), "l"(x));  // x - round(x)
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q) : "l"(c3), "l"(f), "l"(c2));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q) : "l"(q), "l"(f), "l"(c1));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q) : "l"(q), "l"(f), "l"(c0));
  uint32_t r0, r1, q0, q1;
  asm("mov.b64 {%0, %1}, %2;" : "=r"(r0), "=r"(r1) : "l"(r));
  asm("mov.b64 {%0, %1}, %2;" : "=r"(q0), "=r"(q1) : "l"(q));
  p0 = __uint_as_float(q0 + (r0 << 23));
  p1 = __uint_as_float(q1 + (r1 << 23));
}
__device__ __forceinline__ void unpack64(uint64_t v, uint32_t& lo, uint32_t& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t pack64(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}
// arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// 32 TMEM lanes (this warp's) x 32 consecutive 32-bit columns -> 32 registers per thread
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_ld2(uint32_t taddr, uint32_t& r0, uint32_t& r1) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(taddr));
}
__device__ __forceinline__ void tmem_st2(uint32_t taddr, uint32_t r0, uint32_t r1) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};" ::"r"(taddr), "r"(r0), "r"(r1) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Bounded wait that also gives up when another role has raised the abort flag.  Called by whole
// warps; the answer is the same for every lane (the tcgen05 instructions that follow are .aligned).
__device__ __forceinline__ bool umma_wait(uint64_t* bar, uint32_t parity, volatile int* abort) {
  bool ok = false;
  for (int i = 0; i < (1 << 18); ++i) {
    if (mbar_try_wait(bar, parity)) {
      ok = true;
      break;
    }
    if (*abort) break;
    if (i >= 8) __nanosleep(i > 64 ? 256 : kSoftmaxBackoffNs);  // (the first probes back to back: most waits are nearly over)
  }
  if (!ok) *abort = 1;
  return __all_sync(0xffffffffu, ok);
}


// ---- the two MMA issuers: warp 9 issues every QK, warp 10 every PV ----
// Chunk i of this CTA's range (counted over the whole range, not per unit part) belongs to softmax
// group i & 1 and uses that group's score and probability buffers.
//   QK issuer:  wait K/V of chunk i, wait until the group has taken the scores of its previous chunk
//               into registers, issue QK(i)
//   PV issuer:  wait P(i), issue PV(i), release the ring stage and the group's O / P
// so a group's next scores are computed while it works on the current ones.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024 B, version 1, 128-byte swizzle

// The issuer warps run their loops with all 32 lanes in step and one elected lane issuing: every value
// an MMA takes (descriptors, tensor-memory addresses) then depends only on votes and loop counters, which
// the compiler can keep in the uniform datapath the instruction reads its operands from.  With a single
// lane running the loop they lived in ordinary registers and each instruction paid for moving them
// over (≈85 cycles per MMA measured, against 32 of tensor-pipe time).
__device__ __forceinline__ bool issuer_wait(const UmmaCtx& c, uint64_t* bar, uint32_t parity) {
  for (int k = 0; k < (1 << 20); ++k) {
    if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
    if ((k & 15) == 15 && __any_sync(0xffffffffu, *c.abort != 0)) break;
  }
  *c.abort = 1;
  return false;
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

// Narrow form: mine = 0 / 1, this warp issues the QK of group A's / B's chunks (the loop's fixed cost -
// barrier waits, votes, fences, the commit - is about as long as the MMAs themselves, and one warp walking
// every chunk paced the whole pipeline).
// Wide form (W): warp 9 issues both tiles' QK of every chunk: tile A's Q from tensor memory into S_A, tile B's
// from shared memory into S_B.
template <int D, bool W>
__device__ __forceinline__ void umma_issue_qk(const UmmaCtx& c, uint32_t tmem, int lane, int mine) {
  constexpr int HALF_B = kChunk * 128;
  constexpr uint32_t IDESC_QK1 = umma_idesc(kChunk, false);
  // Ring layout: [K column block 0 of every stage][K column block 1 ...][V of every stage].
  // Descriptors differ from one instruction to the next only in the start-address field (units of
  // 16 bytes): everything else is folded into constants.
  const uint32_t k_lo0 = (smem_u32(c.ring) >> 4) | (1u << 16);  // K-major: LBO unused (1)
  const uint32_t k_half = (uint32_t)c.n_stages * (HALF_B >> 4);  // from one 64-column block of K to the next
  const uint32_t tQ = tmem + kTmemQ;  // 16 elements of every row per MMA: 8 columns
  const uint32_t q_lo = (smem_u32(c.qsw) >> 4) | (1u << 16);  // (wide form: tile B's Q, K-major in shared memory)
  constexpr int QHALF = kUmmaRows * 128;
  const bool leader = elect_one();
  int s = 0, ph = 0;       // ring stage / its phase
  int part = 0, left = 0;  // chunks left in the current unit part
  int used_a = 0, used_b = 0;  // QKs issued into S_A / S_B
  for (int i = 0; i < c.n_my;) {
    if (!issuer_wait(c, &c.full_bar[s], ph)) break;
    if (__all_sync(0xffffffffu, left == 0)) {  // first chunk of a unit part: its Q tile
      left = c.metas[s].pad;
      if (__any_sync(0xffffffffu, left < 1) || !issuer_wait(c, c.q_ready, part & 1)) {
        *c.abort = 1;
        break;
      }
      ++part;
    }
    if constexpr (W) {
      // wide form: both tiles' scores of the chunk, A then B.  Tile B's are computed once tile A's rows of
      // the same chunk are in registers, so that the two groups' exp2 phases (one unit per scheduler)
      // coincide less.
      const uint32_t k_lo = k_lo0 + (uint32_t)s * (HALF_B >> 4);
      if (used_a > 0 && !issuer_wait(c, &c.s_free[0], (used_a - 1) & 1)) break;
      tc_fence_after();
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_bf16_ts(tmem, tQ + kk * 8, pack64(k_lo + (kk >> 2) * k_half + (kk & 3) * 2, kDescHi), IDESC_QK1, kk ? 1u : 0u);
        umma_commit(&c.s_full[0]);
      }
      __syncwarp();
      ++used_a;
      if (used_b > 0 && !issuer_wait(c, &c.s_free[1], (used_b - 1) & 1)) break;
      if (!issuer_wait(c, &c.s_free[0], used_b & 1)) break;
      tc_fence_after();
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_bf16(tmem + kChunk, pack64(q_lo + (kk >> 2) * (QHALF >> 4) + (kk & 3) * 2, kDescHi),
                    pack64(k_lo + (kk >> 2) * k_half + (kk & 3) * 2, kDescHi), IDESC_QK1, kk ? 1u : 0u);
        umma_commit(&c.s_full[1]);
      }
      __syncwarp();
      ++used_b;
      ++i;
      --left;
      if (++s == c.n_stages) {
        s = 0;
        ph ^= 1;
      }
      continue;
    }
    const int g = i & 1;
    if (g == mine) {
      // narrow form: the chunk belongs to this issuer's group (the other issuer's chunks only move the
      // ring position along).  Pairing two chunks per QK (N = 128 over S_A and S_B) was tried in three
      // forms - always, when the partner costs no waiting, never - and never is the fastest on verify and
      // prefill tiles alike.
      const int used_g = g ? used_b : used_a;
      if (used_g > 0 && !issuer_wait(c, &c.s_free[g], (used_g - 1) & 1)) break;
      tc_fence_after();  // the tcgen05.ld that read this buffer are done
      const uint32_t k_lo = k_lo0 + (uint32_t)s * (HALF_B >> 4);
      const uint32_t tS = tmem + (uint32_t)g * kChunk;
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_bf16_ts(tS, tQ + kk * 8, pack64(k_lo + (kk >> 2) * k_half + (kk & 3) * 2, kDescHi), IDESC_QK1, kk ? 1u : 0u);
        umma_commit(&c.s_full[g]);
      }
      __syncwarp();
      if (g == 0) ++used_a;
      else ++used_b;
    }
    ++i;
    --left;
    if (++s == c.n_stages) {
      s = 0;
      ph ^= 1;
    }
  }
  // nothing may still be writing tensor memory when it is handed back
  uint64_t* const drain = mine == 1 ? c.drain_b : &c.drain[0];
  if (leader) {
    umma_commit(drain);
    for (int k = 0; k < (1 << 20) && !mbar_try_wait(drain, 0); ++k) __nanosleep(64);
  }
  __syncwarp();
}

// mine: -1 = every PV (narrow form); 0 / 1 = group A's / B's of every chunk (wide form: the two groups do
// not wait for one another anywhere, the ring stage goes back once both PVs have read it)
template <int D, bool W>
__device__ __forceinline__ void umma_issue_pv(const UmmaCtx& c, uint32_t tmem, int lane, int mine) {
  constexpr int KVB = kChunk * D * 2, HALF_B = kChunk * 128;
  constexpr uint32_t IDESC_PV = umma_idesc(D, true);
  // V of stage s sits behind the K blocks of all stages; MN-major: LBO = next 64 columns
  const uint32_t v_lo0 = ((smem_u32(c.ring) + (uint32_t)c.n_stages * KVB) >> 4) | ((uint32_t)(HALF_B >> 4) << 16);
  const bool leader = elect_one();
  int s = 0, ph = 0;
  int left = 0, j = 0;   // chunks left in / done of the current unit part
  int used_a = 0, used_b = 0;  // PVs issued for group A / B
  for (int i = 0; i < c.n_my; ++i) {
    if (__all_sync(0xffffffffu, left == 0)) {  // first chunk of a unit part: how many chunks it has
      if (!issuer_wait(c, &c.full_bar[s], ph)) break;
      left = c.metas[s].pad;
      j = 0;
      if (__any_sync(0xffffffffu, left < 1)) {
        *c.abort = 1;
        break;
      }
    }
    --left;
    const uint32_t v_lo = v_lo0 + (uint32_t)s * (KVB >> 4);
    bool ok = true;
    // narrow: the chunk's group; wide: both groups, A then B
    {
      const int w = W ? mine : (i & 1);
      if (!issuer_wait(c, &c.p_full[w], (w ? used_b : used_a) & 1)) {
        ok = false;
        break;
      }
      tc_fence_after();  // P was written with tcgen05.st
      const uint32_t tO = tmem + kTmemO + (uint32_t)w * 128, tP = tmem + kTmemP + (uint32_t)w * 32;
      const uint32_t acc0 = (W ? j < 1 : j < 2) ? 0u : 1u;  // a group's first chunk of the part overwrites O
      if (leader) {
        umma_bf16_ts(tO, tP, pack64(v_lo, kDescHi), IDESC_PV, acc0);
#pragma unroll
        for (int k = 1; k < 4; ++k)  // 16 keys per instruction
          umma_bf16_ts(tO, tP + k * 8, pack64(v_lo + k * (2048 >> 4), kDescHi), IDESC_PV, 1u);
        umma_commit(&c.empty_bar[s]);  // K and V of this stage have been consumed (wide form: by this group)
        umma_commit(&c.o_full[w]);                          // O_w holds the chunk; P_w may be rewritten
      }
      __syncwarp();
      if (w) ++used_b;
      else ++used_a;
    }
    if (!ok) break;
    ++j;
    if (++s == c.n_stages) {
      s = 0;
      ph ^= 1;
    }
  }
  uint64_t* const drain = mine == 1 ? c.drain_b : &c.drain[1];
  if (leader) {
    umma_commit(drain);
    for (int k = 0; k < (1 << 20) && !mbar_try_wait(drain, 0); ++k) __nanosleep(64);
  }
  __syncwarp();
}

// Merge of a unit's partials by its last arriver (all softmax threads; every partial is in the
// workspace).  A thread owns four adjacent output elements at a time and keeps the loads of two such
// groups times four partials in flight: the loop is bound by L2 latency, not by arithmetic.
template <int D, bool W>
__device__ __forceinline__ void umma_merge(const MmaParams& p, const ResMeta& rm, int t) {
  constexpr int MR = W ? 2 * kUmmaRows : kUmmaRows, REC = MR * (D + 2), V4 = D / 4, U = 2;
  const int G = p.G, total = rm.live * V4;
  for (int e0 = t; e0 < total; e0 += kUmmaSoftmaxThreads * U) {
    int row[U], col[U];
    float M[U], den[U];
    float4 num[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int e = min(e0 + u * kUmmaSoftmaxThreads, total - 1);  // (a clamped duplicate is not stored)
      row[u] = e / V4;
      col[u] = (e - row[u] * V4) * 4;
      M[u] = -INFINITY;
      den[u] = 0.f;
      num[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int c0 = 0; c0 < rm.parts; c0 += 4) {
      float mc[U][4], dc[U][4];
      float4 nn[U][4];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int c = c0 + k;
          mc[u][k] = -INFINITY;
          dc[u][k] = 0.f;
          nn[u][k] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (c < rm.parts) {
            const float* r = p.parts + ((size_t)(rm.first_cta + c) * 2 + (c == 0 ? rm.first_slot : 0)) * REC;
            mc[u][k] = __ldcg(r + MR * D + row[u]);
            dc[u][k] = __ldcg(r + MR * D + MR + row[u]);
            nn[u][k] = __ldcg(reinterpret_cast<const float4*>(r + row[u] * D + col[u]));
          }
        }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float Mn = fmaxf(M[u], mc[u][k]);
          if (Mn != -INFINITY) {
            const float a = (M[u] == -INFINITY) ? 0.f : fast_exp2(M[u] - Mn);
            const float f = (mc[u][k] == -INFINITY) ? 0.f : fast_exp2(mc[u][k] - Mn);
            num[u].x = num[u].x * a + nn[u][k].x * f;
            num[u].y = num[u].y * a + nn[u][k].y * f;
            num[u].z = num[u].z * a + nn[u][k].z * f;
            num[u].w = num[u].w * a + nn[u][k].w * f;
            den[u] = den[u] * a + dc[u][k] * f;
            M[u] = Mn;
          }
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (e0 + u * kUmmaSoftmaxThreads >= total) continue;
      const float inv = den[u] > 0.f ? 1.0f / den[u] : 0.f;
      const int rr = rm.r_lo + row[u], sq = rr / G, g = rr - sq * G;
      *reinterpret_cast<uint2*>(p.out + (size_t)rm.b * p.o_sb + (size_t)(rm.h * G + g) * p.o_sh + (size_t)sq * p.o_ss +
                                col[u]) =
          make_uint2(f2_to_bf2(num[u].x * inv, num[u].y * inv), f2_to_bf2(num[u].z * inv, num[u].w * inv));
    }
  }
}

// ---- the softmax warps ----
// Narrow form (W false, 128 query rows per unit): thread (group w, row r) owns query row r for the chunks
// dealt to group w (A: even, B: odd); the two groups' accumulators are merged when the part ends.
// Wide form (W true, 256 query rows per unit): group w owns rows 128 w .. 128 w + 127 and works on every
// chunk - two query tiles share each K/V chunk the CTA fetches, which halves the L2 -> SM traffic per flop
// (with one tile per fetch the launch was pinned at about 5 TB/s of it, sixteen tiles pulling every K/V
// byte).  Tile A's Q sits in tensor memory, tile B's in shared memory.
template <int D, bool W>
__device__ __forceinline__ void umma_softmax(const MmaParams& p, const UmmaCtx& c, uint32_t tmem, int tid) {
  constexpr int MR = W ? 2 * kUmmaRows : kUmmaRows, REC = MR * (D + 2);
  const int wg = tid >> 7, row = tid & 127, lane = tid & 31, G = p.G;
  const int urow = W ? tid : row;  // the row inside the unit
  const uint32_t t_lane = tmem + ((uint32_t)(row & ~31) << 16);  // this warp's 32 TMEM lanes
  const uint32_t tO = t_lane + kTmemO + (uint32_t)wg * 128, tOo = t_lane + kTmemO + (uint32_t)(wg ^ 1) * 128;
  const float scale = p.scale_log2;
  int cnt = 0;  // chunks this group has worked on (the phase of its barriers)
  int n_pub = 0, n_xch = 0;
  auto group_sync = [&]() -> bool {  // all softmax threads meet (bounded, unlike bar.sync)
    mbar_arrive(c.pub);
    bool ok = false;
    for (int k = 0; k < 4096 && !ok; ++k) ok = mbar_try_wait(c.pub, n_pub & 1);  // everyone is about to arrive
    ok = __all_sync(0xffffffffu, ok) || umma_wait(c.pub, n_pub & 1, c.abort);
    ++n_pub;
    return ok;
  };

  for (int i0 = 0; i0 < c.n_my;) {
    // ---- new unit part: its record, this thread's share of the Q tile ----
    if (!umma_wait(&c.full_bar[i0 % c.n_stages], (i0 / c.n_stages) & 1, c.abort)) return;
    ResMeta fin;
    int n_part, kvs, lim, tok0_part;
    bool live;
    __nv_bfloat16* out_row;
    {
      const MetaM* meta = &c.metas[i0 % c.n_stages];
      const int R = meta->R, r_lo = meta->r_lo, kv_len = meta->kv_len, S = meta->S;
      kvs = meta->kvs;
      tok0_part = meta->tok0;
      n_part = meta->pad;
      fin.b = meta->b;
      fin.h = meta->h;
      fin.r_lo = r_lo;
      fin.live = min(MR, R - r_lo);
      fin.mode = meta->mode;
      fin.parts = meta->parts;
      fin.first_cta = meta->first_cta;
      fin.first_slot = meta->first_slot;
      fin.unit = meta->unit;
      const int r = r_lo + urow;
      live = r < R;
      const int sq = r / G, g = r - sq * G;
      lim = live ? (p.causal ? kv_len - S + sq + 1 : kv_len) : 0;  // first key this row does NOT see
      const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t)fin.b * p.q_sb + (size_t)(fin.h * G + g) * p.q_sh +
                                                        (size_t)sq * p.q_ss);
      out_row = p.out + (size_t)fin.b * p.o_sb + (size_t)(fin.h * G + g) * p.o_sh + (size_t)sq * p.o_ss;
      if constexpr (!W) {
        // each group stores half of the row: D / 2 elements = D / 4 columns (a 16-byte piece is four columns)
        uint32_t qv[D / 4];
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint4 v = live ? __ldg(src + wg * (D / 16) + k) : make_uint4(0, 0, 0, 0);
          qv[4 * k] = v.x; qv[4 * k + 1] = v.y; qv[4 * k + 2] = v.z; qv[4 * k + 3] = v.w;
        }
        const uint32_t tQ = t_lane + kTmemQ + (uint32_t)wg * (D / 4);
        if constexpr (D == 128) tmem_st32(tQ, qv);
        else tmem_st16(tQ, qv);
        tmem_wait_st();
      } else if (wg == 0) {
        // tile A: the whole row into tensor memory, D / 2 columns
#pragma unroll
        for (int hq = 0; hq < 2; ++hq) {
          uint32_t qv[D / 4];
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint4 v = live ? __ldg(src + hq * (D / 16) + k) : make_uint4(0, 0, 0, 0);
            qv[4 * k] = v.x; qv[4 * k + 1] = v.y; qv[4 * k + 2] = v.z; qv[4 * k + 3] = v.w;
          }
          const uint32_t tQ = t_lane + kTmemQ + (uint32_t)hq * (D / 4);
          if constexpr (D == 128) tmem_st32(tQ, qv);
          else tmem_st16(tQ, qv);
        }
        tmem_wait_st();
      } else {
        // tile B: the row's 16-byte pieces into shared memory at their swizzled places (K-major, 128-byte swizzle)
        unsigned char* qrow = c.qsw + row * 128;
#pragma unroll
        for (int cc = 0; cc < D / 8; ++cc) {
          const uint4 v = live ? __ldg(src + cc) : make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(qrow + (cc >> 3) * (kUmmaRows * 128) + (((cc & 7) ^ (row & 7)) << 4)) = v;
        }
        fence_proxy_async();  // generic-proxy writes before the tensor core's async-proxy reads
      }
      tc_fence_before();    // (this thread's reads of O for the previous part are done as well)
      __syncwarp();
      if (lane == 0) mbar_arrive(c.q_ready);
    }
    if (n_part < 1) return;
    const bool warp_live = (urow & ~31) < fin.live;  // a warp of padding rows only keeps the barriers in step
    float m_used = -INFINITY, l = 0.f;

    // narrow: this group takes the chunks whose index in the CTA's range has its parity; wide: every chunk
    const int j_first = W ? 0 : (i0 ^ wg) & 1;
    constexpr int j_step = W ? 1 : 2;
    // With whole pages per chunk every chunk of a part starts chunk_tokens after the one before and
    // the row's own limit already bounds what it holds: nothing of the chunk's record is needed, and
    // neither is a wait for its K/V to land.
    const bool uniform_chunks = p.pages_per_chunk > 0;
    for (int j = j_first; j < n_part; j += j_step) {
      const int i = i0 + j;
      const uint32_t tS = t_lane + (uint32_t)wg * kChunk, tP = t_lane + kTmemP + (uint32_t)wg * 32;
      int rows = p.chunk_tokens, tok0 = tok0_part + j * p.chunk_tokens;
      if (!uniform_chunks) {
        const int s = i % c.n_stages;
        if (!umma_wait(&c.full_bar[s], (i / c.n_stages) & 1, c.abort)) return;
        rows = c.metas[s].rows;
        tok0 = c.metas[s].tok0;
      }
      if (!umma_wait(&c.s_full[wg], cnt & 1, c.abort)) return;
      tc_fence_after();
      if (warp_live) {
        // ---- the row's 64 scores: TMEM -> registers ----
        uint32_t sr[2][32];
        tmem_ld32(tS, sr[0]);
        tmem_ld32(tS + 32, sr[1]);
        tmem_wait_ld();
        // the scores are in registers: the buffer goes back to the QK issuer at once
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&c.s_free[wg]);
        const int lo = max(0, kvs - tok0), hi = min(rows, lim - tok0);  // visible keys of the chunk: [lo, hi)
        // (Rows of padding need no mask: their Q is zero, their scores are finite and nothing of them
        // is ever stored - a warp of a few live rows would otherwise mask on every chunk.)
        if (!__all_sync(0xffffffffu, !live || (lo <= 0 && hi >= kChunk))) {
          const unsigned span = hi > lo ? (unsigned)(hi - lo) : 0u;
#pragma unroll
          for (int k = 0; k < 64; ++k)
            if ((unsigned)(k - lo) >= span) sr[k >> 5][k & 31] = 0xff800000u;  // -inf
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int k = 0; k < 32; ++k)
          mx4[k & 3] = max3(mx4[k & 3], __uint_as_float(sr[k >> 4][(2 * k) & 31]), __uint_as_float(sr[k >> 4][(2 * k + 1) & 31]));
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale;  // scale > 0
        // ---- running maximum; O is rescaled only when some row of the warp moved by more than 2^8 ----
        const bool grow = mx > m_used + kLazyRescale;
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = grow ? mx : m_used;
          const float alpha = grow ? ((m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new)) : 1.f;
          if (j > j_first) {  // O holds the sum of the group's earlier chunks of this part
            if (!umma_wait(&c.o_full[wg], (cnt - 1) & 1, c.abort)) return;
            tc_fence_after();
#pragma unroll
            for (int d0 = 0; d0 < D; d0 += 16) {
              uint32_t ov[16];
              tmem_ld16(tO + d0, ov);
              tmem_wait_ld();
#pragma unroll
              for (int k = 0; k < 16; ++k) ov[k] = __float_as_uint(__uint_as_float(ov[k]) * alpha);
              tmem_st16(tO + d0, ov);
            }
            tmem_wait_st();
          }
          l *= alpha;
          m_used = m_new;
        }
        // ---- P = 2^(s * scale - m), row sum, bf16 pairs into the group's P buffer ----
        const float ne = (m_used == -INFINITY) ? 0.f : -m_used;
        const uint64_t scale2 = pack64(__float_as_uint(scale), __float_as_uint(scale));
        const uint64_t ne2 = pack64(__float_as_uint(ne), __float_as_uint(ne));
        uint64_t l2[2] = {0ull, 0ull};
        uint32_t pk[2][16];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            uint32_t x0, x1;
            unpack64(fma2(pack64(sr[hf][2 * k], sr[hf][2 * k + 1]), scale2, ne2), x0, x1);
            float p0, p1;
            if (W && kWidePolyEvery > 0 && (k % (kWidePolyEvery > 0 ? kWidePolyEvery : 1)) == kWidePolyEvery - 1) {
              exp2_poly2(__uint_as_float(x0), __uint_as_float(x1), p0, p1);
            } else {
              p0 = fast_exp2(__uint_as_float(x0));
              p1 = fast_exp2(__uint_as_float(x1));
            }
            l2[k & 1] = add2(l2[k & 1], pack64(__float_as_uint(p0), __float_as_uint(p1)));
            pk[hf][k] = f2_to_bf2(p0, p1);
          }
          if (hf == 0) {
            // The PV of the group's previous chunk has to have read the buffer (its completion is o_full's
            // phase) before the first store; asked for here, half a row's arithmetic after the scores came,
            // the answer is there without waiting.
            if (cnt > 0) {
              if (!umma_wait(&c.o_full[wg], (cnt - 1) & 1, c.abort)) return;
              tc_fence_after();
            }
          }
          tmem_st16(tP + hf * 16, pk[hf]);
        }
        {
          uint32_t a0, a1, b0, b1;
          unpack64(l2[0], a0, a1);
          unpack64(l2[1], b0, b1);
          l += (__uint_as_float(a0) + __uint_as_float(a1)) + (__uint_as_float(b0) + __uint_as_float(b1));
        }
        tmem_wait_st();
      }
      else {
        // A warp of padding rows keeps the barriers in step - and in order: its arrival for this chunk's
        // P must not reach the barrier while the phase of the group's previous chunk is still open
        // (the scores of the next chunk can be there before the live warps have finished this one).
        __syncwarp();
        if (lane == 0) mbar_arrive(&c.s_free[wg]);
        if (cnt > 0 && !umma_wait(&c.o_full[wg], (cnt - 1) & 1, c.abort)) return;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&c.p_full[wg]);
      ++cnt;
    }

    // ================= end of a unit part =================
    float M = m_used, den = l;
    float* rec = p.parts + ((size_t)c.cta * 2 + (fin.mode == 2 ? 1 : 0)) * REC;
    if constexpr (W) {
      // wide: the group's own rows, the whole head dimension; nothing to merge inside the CTA
      if (!umma_wait(&c.o_full[wg], (cnt - 1) & 1, c.abort)) return;
      tc_fence_after();
      if (warp_live) {
        const float inv = den > 0.f ? 1.0f / den : 0.f;
        const float s_m = fin.mode == 0 ? inv : 1.f;
#pragma unroll
        for (int d0 = 0; d0 < D; d0 += 32) {
          uint32_t om[32];
          float v[32];
          tmem_ld32(tO + d0, om);
          tmem_wait_ld();
#pragma unroll
          for (int k = 0; k < 32; ++k) v[k] = __uint_as_float(om[k]) * s_m;
          if (live) {
            if (fin.mode == 0) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4)
                *reinterpret_cast<uint4*>(out_row + d0 + q4 * 8) =
                    make_uint4(f2_to_bf2(v[q4 * 8], v[q4 * 8 + 1]), f2_to_bf2(v[q4 * 8 + 2], v[q4 * 8 + 3]),
                               f2_to_bf2(v[q4 * 8 + 4], v[q4 * 8 + 5]), f2_to_bf2(v[q4 * 8 + 6], v[q4 * 8 + 7]));
            } else {
#pragma unroll
              for (int q4 = 0; q4 < 8; ++q4)
                *reinterpret_cast<float4*>(rec + urow * D + d0 + q4 * 4) =
                    make_float4(v[q4 * 4], v[q4 * 4 + 1], v[q4 * 4 + 2], v[q4 * 4 + 3]);
            }
          }
        }
      }
    } else {
      const bool has_mine = j_first < n_part, has_other = (j_first ^ 1) < n_part;  // (a part of one chunk leaves a group empty-handed)
      if (has_mine && !umma_wait(&c.o_full[wg], (cnt - 1) & 1, c.abort)) return;
      // Each row's (reference maximum, sum) crosses to the other group through tensor memory: columns 0
      // and 1 of the group's own score buffer, which holds nothing any more (the scores of its last chunk
      // are long in registers; the next QK into the buffer waits for the next part's Q).  Both groups'
      // warp w own the same 32 TMEM lanes, so no shared memory is needed.
      if (has_mine) {
        tmem_st2(t_lane + (uint32_t)wg * kChunk, __float_as_uint(m_used), __float_as_uint(l));
        tmem_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(c.xch);
      if (!umma_wait(c.xch, n_xch & 1, c.abort)) return;
      ++n_xch;
      tc_fence_after();
      float m_o = -INFINITY, l_o = 0.f;
      if (has_other) {
        uint32_t xm, xl;
        tmem_ld2(t_lane + (uint32_t)(wg ^ 1) * kChunk, xm, xl);
        tmem_wait_ld();
        m_o = __uint_as_float(xm);
        l_o = __uint_as_float(xl);
      }
      M = fmaxf(m_used, m_o);
      const float f_m = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - M);
      const float f_o = (m_o == -INFINITY) ? 0.f : fast_exp2(m_o - M);
      den = l * f_m + l_o * f_o;
      // group A takes the lower half of the head dimension, group B the upper half
      if (warp_live) {
        const float inv = den > 0.f ? 1.0f / den : 0.f;
        const float s_m = fin.mode == 0 ? f_m * inv : f_m, s_o = fin.mode == 0 ? f_o * inv : f_o;
  #pragma unroll
        for (int d0 = wg * (D / 2); d0 < (wg + 1) * (D / 2); d0 += 32) {
          float v[32];
  #pragma unroll
          for (int k = 0; k < 32; ++k) v[k] = 0.f;
          if (has_mine) {
            uint32_t om[32];
            tmem_ld32(tO + d0, om);
            tmem_wait_ld();
  #pragma unroll
            for (int k = 0; k < 32; ++k) v[k] = __uint_as_float(om[k]) * s_m;
          }
          if (has_other) {
            uint32_t oo[32];
            tmem_ld32(tOo + d0, oo);
            tmem_wait_ld();
  #pragma unroll
            for (int k = 0; k < 32; ++k) v[k] = fmaf(__uint_as_float(oo[k]), s_o, v[k]);
          }
          if (live) {
            if (fin.mode == 0) {
  #pragma unroll
              for (int q4 = 0; q4 < 4; ++q4)
                *reinterpret_cast<uint4*>(out_row + d0 + q4 * 8) =
                    make_uint4(f2_to_bf2(v[q4 * 8], v[q4 * 8 + 1]), f2_to_bf2(v[q4 * 8 + 2], v[q4 * 8 + 3]),
                               f2_to_bf2(v[q4 * 8 + 4], v[q4 * 8 + 5]), f2_to_bf2(v[q4 * 8 + 6], v[q4 * 8 + 7]));
            } else {
  #pragma unroll
              for (int q4 = 0; q4 < 8; ++q4)
                *reinterpret_cast<float4*>(rec + row * D + d0 + q4 * 4) =
                    make_float4(v[q4 * 4], v[q4 * 4 + 1], v[q4 * 4 + 2], v[q4 * 4 + 3]);
            }
          }
        }
      }
    }
    tc_fence_before();
    i0 += n_part;
    if (fin.mode == 0) continue;
    // cut unit: the fp32 partial is in the workspace; arrival count, merge by the last arriver
    if (live && (W || wg == 0)) {
      rec[MR * D + urow] = M;
      rec[MR * D + MR + urow] = den;
    }
    __threadfence();
    if (!group_sync()) return;
    int* const flag = c.flag + (n_pub & 2 ? 1 : 0);  // two slots in turn: no third meeting to protect a rewrite
    if (tid == 0) {
      const int old = atomicAdd(&p.unit_count[fin.unit], 1);
      const int is_last = (old == fin.parts - 1);
      if (is_last) p.unit_count[fin.unit] = 0;  // ready for the next launch
      *flag = is_last;
    }
    if (!group_sync()) return;
    const int is_last = *flag;
    if (is_last) {
      __threadfence();
      umma_merge<D, W>(p, fin, tid);
    }
  }
}

// Entry of warps 0..7 and 9..11 of a CTA that has work: warp 9 owns the tensor memory and issues QK MMAs
// (warp 11 those of group B's chunks on full tiles), warp 10 the PV MMAs, warps 0..7 are the two softmax groups.  Every wait inside is bounded and every path ends at
// the barrier in front of the deallocation: a CTA never exits holding tensor memory.
template <int D, bool W>
__device__ __forceinline__ void umma_consumer(const MmaParams& p, const UmmaCtx& c, int tid) {
  const int warp = tid >> 5, lane = tid & 31;
  const bool owner = warp == kUmmaQkWarp;
  if (owner) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(c.tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  asm volatile("bar.sync 3, 352;" ::: "memory");
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(c.tmem_slot);
  if (warp == kUmmaQkWarp) umma_issue_qk<D, W>(c, tmem, lane, 0);
  else if (warp == kUmmaWarpB) {
    if (W) umma_issue_pv<D, W>(c, tmem, lane, 1);
    else umma_issue_qk<D, W>(c, tmem, lane, 1);
  } else if (warp == kUmmaPvWarp) umma_issue_pv<D, W>(c, tmem, lane, W ? 0 : -1);
  else umma_softmax<D, W>(p, c, tmem, tid);
  if (lane == 0 && *c.abort) raise_status(p.kv.status, PACE_DEV_WAIT_TIMEOUT);
  tc_fence_before();
  asm volatile("bar.sync 3, 352;" ::: "memory");
  if (owner) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

}  // namespace
}  // namespace pace
