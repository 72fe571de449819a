// Block-sparse causal prefill (attention sink + per-head sliding window) on tcgen05 / TMEM / TMA.
//
// The unit of work is a 256-row query super-tile of one (batch, head): two 128-row tiles A and B that share
// every K/V tile brought into shared memory.  The kernel comes in two forms (a template flag; the launcher
// chooses by shape): persistent — one thread block per SM working through units handed out by an atomic
// counter, heaviest first — and one block per unit.  Roles of a block:
//   warps 0-3  softmax of tile A, warps 4-7 softmax of tile B: thread r owns query row r of its
//              tile (= TMEM lane r).  Per KV block it loads its S row from TMEM, computes the
//              exponentials against a lazily updated max, writes P (fp16/bf16, two per 32-bit
//              column) over the first half of the S buffer the row came from, rescales O in TMEM
//              when the max moved, and finally runs the epilogue
//   warp  8    scheduler + TMA producer (one lane): fetches the next super-tile, publishes it to the other
//              roles through a two-entry ring (persistent form), loads both Q tiles, then K and V tiles of 64
//              tokens through two rings of shared-memory stages.  It runs ahead of the others: the next
//              super-tile's Q and first K/V tiles arrive while the softmax warps are still in the epilogue of
//              this one
//   warp  9,10 MMA issuers of tile A and tile B (warp 9 owns the TMEM allocation):
//              S = Q K^T (M128 N64 K128, Q and K from shared memory), O += P V (M128 N128 K64,
//              P from TMEM, V from shared memory as an MN-major operand).  The whole warp runs the
//              issuer loop with warp-uniform control flow (operands stay in uniform registers) and
//              one elected lane issues; the KV blocks a tile takes part in are two index ranges in
//              closed form.
// Each tile has two S/P buffers in TMEM.  On the tensor core its order is S(0), S(1), then per step
// i: [softmax turns S(i) into P(i)] -> O += P(i) V(i) -> S(i+2), the last one into the buffer P(i)
// was read from: MMAs of one issuing thread execute in order, so no barrier guards the buffers,
// and S runs a whole step ahead of the exponentials.  The same order carries over from one super-tile to
// the next: its S(0) and S(1) are issued right behind the last O += P V, and the first O += P V of the
// next super-tile (which overwrites O) waits for a P that the softmax threads only produce after their
// epilogue has read O.  Shared-memory stages go back to the producer through tcgen05.commit.  Only the
// 64-token KV blocks inside "sink U band" of the super-tile are loaded; a tile skips the blocks only the
// other tile sees, and only the (at most three) edge blocks of a tile get an element mask.
//
// Every mbarrier is used with a running count kept by each role (stage or buffer = count mod ring size,
// parity = the next bit), so phases carry over from super-tile to super-tile.
//
// The mask (MoA/kernels/block_sparse_attention_prefill.py:558-580): query block bi = row/64 sees
// KV block j iff j <= bi and (j < sink_blocks[h] or j >= bi + 1 - local_blocks[h]); inside a
// block: key <= query and key < N.
//
// Every wait on an mbarrier is bounded: when it runs out the block sets an abort flag, records a
// code in the status words, drains, frees its TMEM and returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <type_traits>

#include "common.cuh"

namespace moa {
namespace {

constexpr int kD = 128;            // largest head_dim (shared-memory and TMEM layout are sized for it; 64 uses half)
constexpr int kBM = 128;           // query rows per tile (two tiles per block)
constexpr int kBN = 64;            // KV tokens per tile (= the mask's block size)
constexpr int kStages = 4;         // depth of the K ring and of the V ring (power of two)
constexpr int kSoftmaxThreads = 128;  // per tile
constexpr int kThreads = 352;
constexpr uint32_t kTmemCols = 512;
// TMEM columns: O_A [0,128) O_B [128,256); S/P buffers of tile A [256,320) [320,384), of tile B [384,448) [448,512)
__host__ __device__ constexpr uint32_t col_o(int x) { return (uint32_t)x * 128u; }
__host__ __device__ constexpr uint32_t col_s(int x, int buf) { return 256u + (uint32_t)x * 128u + (uint32_t)buf * 64u; }

constexpr int kQBytes = kBM * kD * 2;       // 32 KiB per Q tile (two 16 KiB halves: dims 0-63, 64-127)
constexpr int kKBytes = kBN * kD * 2;       // 16 KiB per K or V tile (two 8 KiB halves)
constexpr int kSmemQ = 0;
constexpr int kSmemK = kSmemQ + 2 * kQBytes;
constexpr int kSmemV = kSmemK + kStages * kKBytes;
constexpr int kSmemCtl = kSmemV + kStages * kKBytes;
constexpr int kSmemStage = kSmemCtl + 512;  // epilogue staging: 32 rows of 128 B for each of the 8 softmax warps
constexpr int kStageBytes = 32 * 128;
constexpr int kSmemBytes = kSmemStage + 8 * kStageBytes + 1024;  // + slack for 1024-byte alignment
static_assert(kSmemBytes <= 227 * 1024, "shared memory of one block");

// the running max is only moved when a block exceeds it by more than this (log2 units)
constexpr float kLazyMaxSlack = 8.f;
constexpr long long kWaitLimitCycles = 4000000000ll;  // about 2 s of SM clock: far above any legitimate wait
constexpr uint64_t kWaitLimitNs = 2000000000ull;      // same bound for the drain loops of the abort path

// status codes written to status[0] when a wait gives up
enum { kWaitQ = 1, kWaitKFull = 2, kWaitKEmpty = 3, kWaitS = 4, kWaitP = 5, kWaitPV = 6, kWaitO = 7,
       kWaitVFull = 8, kWaitVEmpty = 9, kWaitLock = 11, kWaitTile = 12, kWaitTileSlot = 13, kWaitQEmpty = 14 };

struct Ctl {
  uint64_t q_full;               // producer -> issuers: both Q tiles of the super-tile are in shared memory
  uint64_t q_empty[2];           // [tile] issuer -> producer: that tile's Q K^T of the super-tile have all been executed
                                 // (one barrier per issuer: an issuer with nothing to do in the next super-tile arrives
                                 // again at once, and must not be taken for the other one)
  uint64_t k_full[kStages];
  uint64_t v_full[kStages];
  uint64_t k_empty[2][kStages];  // [tile]: that tile is done with the K stage
  uint64_t v_empty[2][kStages];
  uint64_t s_full[2][2];   // [tile][S buffer] tensor core -> softmax: S is in TMEM
  uint64_t p_full[2][2];  // [tile][S/P buffer] softmax -> issuer: P is in TMEM (and O rescaled).  One per buffer: the
                          // softmax threads can be two steps ahead of the issuer, and a single barrier would
                          // then have advanced two phases, which a parity wait cannot tell from none
  uint64_t pv_done[2];  // [tile] tensor core -> softmax: the last but one O += P V has finished (O may be rescaled)
  uint64_t o_full[2];
  uint64_t tile_full[2];   // producer -> everyone: tile_id[slot] holds the next super-tile (or -1: no more)
  uint64_t tile_empty[2];  // everyone -> producer: the slot has been read (count kTileReaders)
  int tile_id[2];
  uint32_t tmem_base;
  int abort;
  int pipe_lock;   // held by the issuer whose batch of MMAs is being queued
};
static_assert(sizeof(Ctl) <= 512, "control block");
constexpr int kTileReaders = 2 + 8;   // one elected lane of each issuer warp, lane 0 of each softmax warp

struct PrefillParams {
  void* out;
  int64_t o_sb, o_sn, o_sh;
  const int32_t* sink_blocks;
  const int32_t* local_blocks;
  int B, H;
  int64_t N;
  float scale_log2;
  int chunk;         // consecutive super-tiles of a head that are handed out together (see tile_coord)
  int nsuper;        // 256-row super-tiles per (batch, head)
  int num_tiles;     // B * H * nsuper
  int32_t* status;   // [0..3] wait report; [4] next super-tile to hand out, [5] blocks that have finished
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait.  Returns false when the block is aborting (this wait or another one gave up).
// The limit is counted with clock64 (a cheap per-SM counter); reading %globaltimer costs far more
// than a typical wait lasts and must stay off this path.
__device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, Ctl* ctl, int32_t* status, int code,
                                            long long limit_cycles = kWaitLimitCycles) {
  const long long t0 = clock64();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 255u) == 0) {
      if (*(volatile int*)&ctl->abort) return false;
      if (clock64() - t0 > limit_cycles) {
        *(volatile int*)&ctl->abort = 1;
        if (atomicCAS(&status[0], 0, code) == 0) {
          status[1] = (int32_t)blockIdx.x;
          status[2] = (int32_t)(blockIdx.y + 65536 * blockIdx.z);
          status[3] = (int32_t)threadIdx.x;
        }
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Ctl* ctl, int32_t* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, ctl, status, code);
}

// One lane of a converged warp (the lowest active one).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// The two issuers take turns on the tensor core: a tile's batch (O += P V, then the S two steps ahead) is
// queued as a whole.  Interleaved MMA by MMA, both tiles' S would complete only when all of both batches has
// run; queued whole, the first tile's S is complete after its own batch, and the tiles drift into opposite
// phases.  Bounded like every other wait.
__device__ __forceinline__ bool pipe_acquire(Ctl* ctl, int32_t* status) {
  const long long t0 = clock64();
  for (uint32_t spin = 1; atomicCAS(&ctl->pipe_lock, 0, 1) != 0; ++spin) {
    if ((spin & 255u) == 0) {
      if (*(volatile int*)&ctl->abort) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        *(volatile int*)&ctl->abort = 1;
        if (atomicCAS(&status[0], 0, kWaitLock) == 0) {
          status[1] = (int32_t)blockIdx.x;
          status[2] = (int32_t)(blockIdx.y + 65536 * blockIdx.z);
          status[3] = (int32_t)threadIdx.x;
        }
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void pipe_release(Ctl* ctl) { atomicExch(&ctl->pipe_lock, 0); }

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem desc]   (A: 128 lanes x K, two 16-bit values per 32-bit column)
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// three-input maximum (one instruction on sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

#define MOA_R32(v) \
  v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], v[8], v[9], v[10], v[11], v[12], v[13], v[14], v[15], v[16], \
  v[17], v[18], v[19], v[20], v[21], v[22], v[23], v[24], v[25], v[26], v[27], v[28], v[29], v[30], v[31]

// 32 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100).
//   K-major operand : rows of 128 B (64 elements of K), 8-row groups 1024 B apart (SBO); LBO unused
//   MN-major operand: rows (one per K index) of 128 B (64 elements of MN), 8-row groups 1024 B
//                     apart (SBO); the next 64 MN elements start LBO bytes further on
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16 with fp32 accumulation.  A and B have separate format fields (0 = fp16,
// 1 = bf16) but must be given the same format: fp16 A (P) with bf16 B (V) raises an illegal-instruction
// error on B200.
__host__ __device__ constexpr uint32_t make_idesc(int is_bf16, int b_mn_major, int M, int N) {
  return (1u << 4) | ((uint32_t)is_bf16 << 7) | ((uint32_t)is_bf16 << 10) | ((uint32_t)b_mn_major << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// KV blocks a query super-tile visits, as a list: entries [0, nA) are blocks 0..nA-1 (sink part),
// entries [nA, nA + nB) are blocks bB, bB+1, ... (band part).
struct TileBlocks {
  int nA, bB, nB;
  __device__ __forceinline__ int count() const { return nA + nB; }
  __device__ __forceinline__ int block(int u) const { return u < nA ? u : bB + (u - nA); }
};
// t_lo, t_hi: first and last 128-row tile of the super-tile
__device__ __forceinline__ TileBlocks tile_blocks(int t_lo, int t_hi, int nb, int sink_b, int local_b) {
  const int hi = min(2 * t_hi + 2, nb);              // blocks [0, hi) are at or below the diagonal
  TileBlocks r;
  r.nA = max(0, min(sink_b, hi));
  r.bB = max(r.nA, 2 * t_lo + 1 - local_b);           // first band block of the first 64 rows
  r.nB = max(0, hi - r.bB);
  return r;
}
// The list entries one 128-row tile t takes part in: [0, s_end) and [b_begin, b_end).
// (Block j is visible to the tile iff j < min(2t+2, nb) and (j < sink or j >= 2t+1-local).)
struct TileSeen {
  int s_end, b_begin, b_end, total;
  __device__ __forceinline__ int entry(int i) const { return i < s_end ? i : b_begin + (i - s_end); }
};
__device__ __forceinline__ TileSeen tile_seen(bool exists, int t, const TileBlocks& tb, int nb, int local_b) {
  TileSeen r;
  const int hi = min(2 * t + 2, nb), lo = 2 * t + 1 - local_b;
  r.s_end = exists ? min(tb.nA, hi) : 0;
  r.b_begin = tb.nA + max(lo, tb.bB) - tb.bB;
  r.b_end = tb.nA + min(hi, tb.bB + tb.nB) - tb.bB;
  if (!exists || tb.nB == 0 || r.b_end < r.b_begin) r.b_end = r.b_begin;
  r.total = r.s_end + (r.b_end - r.b_begin);
  return r;
}

// Which (batch, head, super-tile) the n-th handed-out unit is.  A head's super-tiles get heavier towards the end
// of the sequence (until the window is full), so units are handed out from the end of the sequence backwards,
// in chunks of `chunk` consecutive super-tiles per head: chunk by chunk, inside a chunk head by head, inside a
// head from the last super-tile down.  Every head's heavy tiles therefore start early and the launch ends on
// cheap ones (the longest-processing-time order, up to the chunk), while the blocks working at the same time
// still hold neighbouring super-tiles of a head, which share their K/V band in L2.  chunk = 1 interleaves the
// heads completely; chunk = nsuper takes one head after the other.
struct TileCoord {
  int b, h, st;
};
__device__ __forceinline__ TileCoord tile_coord(int unit, const PrefillParams& p) {
  const int heads = p.B * p.H;
  const int per_chunk = heads * p.chunk;              // units in a full chunk
  const int full = p.nsuper / p.chunk;                // full chunks, counted from the end of the sequence
  int k = unit / per_chunk, width = p.chunk, r = unit - k * per_chunk;
  if (k >= full) {                                    // the partial chunk at the start of the sequence
    k = full;
    width = p.nsuper - full * p.chunk;
    r = unit - full * per_chunk;
  }
  const int bh = r / width, j = r - bh * width;
  TileCoord c;
  c.b = bh / p.H;
  c.h = bh - c.b * p.H;
  c.st = p.nsuper - 1 - k * p.chunk - j;
  return c;
}

// Everything a role derives from a super-tile's coordinates.
struct TileWork {
  int b, h, t0, nb, sink_b, local_b, nkv;
  bool active1;       // the second 128-row tile exists
  TileBlocks tb;
};
__device__ __forceinline__ TileWork tile_work(int unit, const PrefillParams& p) {
  const TileCoord c = tile_coord(unit, p);
  TileWork w;
  w.b = c.b;
  w.h = c.h;
  w.t0 = 2 * c.st;
  w.nb = (int)((p.N + kBN - 1) / kBN);
  w.sink_b = p.sink_blocks[c.h];
  w.local_b = p.local_blocks[c.h];
  w.active1 = (int64_t)(w.t0 + 1) * kBM < p.N;
  w.tb = tile_blocks(w.t0, w.active1 ? w.t0 + 1 : w.t0, w.nb, w.sink_b, w.local_b);
  w.nkv = w.tb.count();
  return w;
}

// DH = head_dim, 64 or 128.  The shared-memory and TMEM layout is the one of 128; with 64 only the first
// 64-column panel of every Q/K/V tile and the first 64 O columns are used.
//
// PERSISTENT: the block keeps taking units from the counter until there are none left (the grid is one block per
// SM).  Otherwise the block computes the one unit that is its index (the grid is one block per unit, handed to
// the SMs in order by the hardware) and the loops below run once: the form for long sequences, where a
// super-tile runs for hundreds of steps, the hand-over between units does not matter, and the code the compiler
// makes of the single pass is a few per cent faster per step.
template <typename T, bool OUT_F32, int DH, bool PERSISTENT>
__global__ void __launch_bounds__(kThreads, 1)
moa_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const PrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  Ctl* ctl = reinterpret_cast<Ctl*>(smem + kSmemCtl);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr int NH = DH / 64;                 // 64-column panels per tile
  constexpr int kQPanel = kBM * 128, kKPanel = kBN * 128;   // bytes of one panel
  static_assert(DH == 64 || DH == 128, "head_dim");

  // the block's first unit is its own index: fetch its head's plan while the barriers and TMEM are set up
  const TileWork w_first = tile_work((int)blockIdx.x, p);
  if (warp == 8 && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  if (tid == 0) {
    mbar_init(&ctl->q_full, 1);
    mbar_init(&ctl->q_empty[0], 1);
    mbar_init(&ctl->q_empty[1], 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&ctl->k_full[s], 1);
      mbar_init(&ctl->v_full[s], 1);
      for (int x = 0; x < 2; ++x) {
        mbar_init(&ctl->k_empty[x][s], 1);
        mbar_init(&ctl->v_empty[x][s], 1);
      }
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(&ctl->s_full[x][0], 1);
      mbar_init(&ctl->s_full[x][1], 1);
      mbar_init(&ctl->p_full[x][0], kSoftmaxThreads);
      mbar_init(&ctl->p_full[x][1], kSoftmaxThreads);
      mbar_init(&ctl->pv_done[x], 1);
      mbar_init(&ctl->o_full[x], 1);
      mbar_init(&ctl->tile_full[x], 1);
      mbar_init(&ctl->tile_empty[x], kTileReaders);
    }
    ctl->abort = 0;
    ctl->pipe_lock = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *(volatile uint32_t*)&ctl->tmem_base;

  if (warp == 8) {
    // ------------------------------------------------------------------ scheduler + TMA producer
    if (lane == 0) {
      uint32_t ring = 0;            // K (and V) ring entries of the super-tiles before this one
      uint32_t k_issued = 0, v_issued = 0, q_issued = 0;
      bool ok = true;
      for (uint32_t n = 0; ok; ++n) {
        int unit = (int)blockIdx.x;      // the first unit of a block is its own index
        if (PERSISTENT) {
          if (n > 0) unit = (int)gridDim.x + atomicAdd(&p.status[4], 1);   // later ones come from the counter
          if (unit >= p.num_tiles) unit = -1;
          const int slot = n & 1;
          // Q may be overwritten once both issuers' Q K^T of the previous super-tile have been executed.  This
          // wait comes before the next unit is published: an issuer with nothing to do in it hands Q back at
          // once, and that second arrival must not land before the first one has been seen here.
          if (n > 0) {
            ok = mbar_wait(&ctl->q_empty[0], (n - 1) & 1, ctl, p.status, kWaitQEmpty) &&
                 mbar_wait(&ctl->q_empty[1], (n - 1) & 1, ctl, p.status, kWaitQEmpty);
            if (!ok) break;
          }
          ok = mbar_wait(&ctl->tile_empty[slot], ((n >> 1) & 1) ^ 1, ctl, p.status, kWaitTileSlot);
          if (!ok) break;
          *(volatile int*)&ctl->tile_id[slot] = unit;
          mbar_arrive(&ctl->tile_full[slot]);
          if (unit < 0) break;
        } else if (n > 0) {
          break;
        }
        const TileWork w = (n == 0) ? w_first : tile_work(unit, p);
        // A super-tile that visits no KV block at all (a head without sink and window at the ragged end of the
        // sequence) loads nothing: nobody would wait for its Q, and a copy must never be in flight when the block
        // ends, nor may q_full be armed again before its previous phase has completed.
        if (w.nkv > 0) {
          mbar_expect_tx(&ctl->q_full, 2 * NH * kQPanel);
#pragma unroll
          for (int hf = 0; hf < NH; ++hf) {
            tma_load_4d(smem + kSmemQ + hf * kQPanel, &map_q, &ctl->q_full, 64 * hf, w.t0 * kBM, w.h, w.b);
            tma_load_4d(smem + kSmemQ + kQBytes + hf * kQPanel, &map_q, &ctl->q_full, 64 * hf, (w.t0 + 1) * kBM, w.h, w.b);
          }
          ++q_issued;
        }
        // V lags K by one tile: it is needed one MMA step later.  A stage is reused once both
        // tiles' issuers have handed it back.
        for (int u = 0; ok && u <= w.nkv; ++u) {
          if (u < w.nkv) {
            const uint32_t g = ring + u;
            const int s = g & (kStages - 1);
            const uint32_t par = ((g / kStages) & 1) ^ 1;
            ok = mbar_wait(&ctl->k_empty[0][s], par, ctl, p.status, kWaitKEmpty) &&
                 mbar_wait(&ctl->k_empty[1][s], par, ctl, p.status, kWaitKEmpty);
            if (!ok) break;
            uint8_t* dst = smem + kSmemK + s * kKBytes;
            const int row = w.tb.block(u) * kBN;
            mbar_expect_tx(&ctl->k_full[s], NH * kKPanel);
#pragma unroll
            for (int hf = 0; hf < NH; ++hf) tma_load_4d(dst + hf * kKPanel, &map_k, &ctl->k_full[s], 64 * hf, row, w.h, w.b);
            k_issued = g + 1;
          }
          if (u >= 1) {
            const uint32_t g = ring + u - 1;
            const int s = g & (kStages - 1);
            const uint32_t par = ((g / kStages) & 1) ^ 1;
            ok = mbar_wait(&ctl->v_empty[0][s], par, ctl, p.status, kWaitVEmpty) &&
                 mbar_wait(&ctl->v_empty[1][s], par, ctl, p.status, kWaitVEmpty);
            if (!ok) break;
            uint8_t* dst = smem + kSmemV + s * kKBytes;
            const int row = w.tb.block(u - 1) * kBN;
            mbar_expect_tx(&ctl->v_full[s], NH * kKPanel);
#pragma unroll
            for (int hf = 0; hf < NH; ++hf) tma_load_4d(dst + hf * kKPanel, &map_v, &ctl->v_full[s], 64 * hf, row, w.h, w.b);
            v_issued = g + 1;
          }
        }
        ring += (uint32_t)w.nkv;
      }
      // This block has taken its last unit (or is giving up).  The last block to get here puts the scheduler
      // words back to zero for the next launch — nobody touches them any more — while the others still compute.
      if (PERSISTENT) {
        __threadfence();
        if (atomicAdd(&p.status[5], 1) == (int)gridDim.x - 1) {
          p.status[4] = 0;
          p.status[5] = 0;
        }
      }
      if (*(volatile int*)&ctl->abort) {
        // drain: shared memory must not be released while bulk copies into it are in flight
        const uint64_t tstart = globaltimer_ns();
        for (uint32_t g = k_issued > (uint32_t)kStages ? k_issued - kStages : 0; g < k_issued; ++g) {
          while (!mbar_try_wait(&ctl->k_full[g & (kStages - 1)], (g / kStages) & 1) &&
                 globaltimer_ns() - tstart < kWaitLimitNs) {
          }
        }
        for (uint32_t g = v_issued > (uint32_t)kStages ? v_issued - kStages : 0; g < v_issued; ++g) {
          while (!mbar_try_wait(&ctl->v_full[g & (kStages - 1)], (g / kStages) & 1) &&
                 globaltimer_ns() - tstart < kWaitLimitNs) {
          }
        }
        if (q_issued > 0) {
          while (!mbar_try_wait(&ctl->q_full, (q_issued - 1) & 1) && globaltimer_ns() - tstart < kWaitLimitNs) {
          }
        }
      }
    }
  } else if (warp >= 9) {
    // ------------------------------------------------------------------ MMA issuer of tile x
    // The whole warp runs this code with warp-uniform control flow and values, so that descriptors and
    // addresses can stay in uniform registers; one elected lane issues the MMAs, commits and arrives.
    // (Issued from lane 0 of a divergent branch the same MMAs cost about three times as many cycles each.)
    //
    // Order on the tensor core for this tile: S(0), S(1), then for every step i: O += P(i) V(i), S(i+2).
    // S(i+2) goes into the buffer P(i) is read from; MMAs of one thread execute in order, so it cannot
    // overtake that read, and no barrier is needed for the buffer.
    const int x = warp - 9;
    constexpr uint32_t idesc_qk = make_idesc(kBf16, 0, kBM, kBN);
    constexpr uint32_t idesc_pv = make_idesc(kBf16, 1, kBM, DH);
    // descriptors differ only in their start-address field (bytes >> 4): build each base once
    const uint64_t q_desc = make_desc(smem_u32(smem + kSmemQ + x * kQBytes), 16, 1024);
    const uint64_t k_desc0 = make_desc(smem_u32(smem + kSmemK), 16, 1024);
    const uint64_t v_desc0 = make_desc(smem_u32(smem + kSmemV), kKBytes / 2, 1024);
    const uint32_t o_tmem = tmem + col_o(x);
    uint64_t* const k_empty = ctl->k_empty[x];
    uint64_t* const v_empty = ctl->v_empty[x];
    uint32_t ring = 0;   // K/V ring entries of the super-tiles before this one
    uint32_t sbase = 0;  // S/P buffers this tile has used before this super-tile
    uint32_t q_loads = 0;  // super-tiles before this one whose Q was loaded (those that visit any KV block)
    bool ok = true;
    auto wait = [&](uint64_t* bar, uint32_t parity, int code) {
      const bool mine = mbar_wait(bar, parity, ctl, p.status, code);
      ok = __all_sync(0xffffffffu, mine);
    };

    for (uint32_t n = 0; ok; ++n) {
      int unit = (int)blockIdx.x;
      if (PERSISTENT) {
        const int slot = n & 1;
        wait(&ctl->tile_full[slot], (n >> 1) & 1, kWaitTile);
        if (!ok) break;
        unit = *(volatile int*)&ctl->tile_id[slot];
        __syncwarp();
        if (elect_one()) mbar_arrive(&ctl->tile_empty[slot]);
        if (unit < 0) break;
      } else if (n > 0) {
        break;
      }
      const TileWork w = (n == 0) ? w_first : tile_work(unit, p);
      const int nkv = w.nkv;
      const TileSeen seen = tile_seen(x == 0 || w.active1, w.t0 + x, w.tb, w.nb, w.local_b);

      // Hand back ring entries [from, to) this tile does not use (rare: at most a few per tile).  The stage
      // must have been filled first, so that the arrives of successive ring rounds cannot run ahead of the
      // producer.
      auto skip_k = [&](int from, int to) {
        for (int e = from; ok && e < to; ++e) {
          const uint32_t g = ring + e;
          const int s = g & (kStages - 1);
          wait(&ctl->k_full[s], (g / kStages) & 1, kWaitKFull);
          if (ok && elect_one()) mbar_arrive(&k_empty[s]);
        }
      };
      auto skip_v = [&](int from, int to) {
        for (int e = from; ok && e < to; ++e) {
          const uint32_t g = ring + e;
          const int s = g & (kStages - 1);
          wait(&ctl->v_full[s], (g / kStages) & 1, kWaitVFull);
          if (ok && elect_one()) mbar_arrive(&v_empty[s]);
        }
      };
      // K and V of the same entries, entry by entry in the order the producer fills them
      auto skip_both = [&](int from, int to) {
        for (int e = from; ok && e < to; ++e) {
          skip_k(e, e + 1);
          skip_v(e, e + 1);
        }
      };
      // the MMAs of S(j) = Q K^T for the tile's j-th entry, into S buffer (sbase + j) & 1 (issuing lane only)
      auto qk_mmas = [&](int j, int s) {
        const uint64_t k_desc = k_desc0 + (uint64_t)(s * (kKBytes >> 4));
        const uint32_t buf = (sbase + (uint32_t)j) & 1u;
        const uint32_t s_tmem = tmem + col_s(x, buf);
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          // 16 dims per step: 32 B inside the swizzle row; dims 64-127 sit in the second half-tile
          const uint32_t half = kk >> 2, off = (kk & 3) * 32;
          tc_mma_ss(s_tmem, q_desc + (uint64_t)((half * (kQBytes / 2) + off) >> 4),
                    k_desc + (uint64_t)((half * (kKBytes / 2) + off) >> 4), idesc_qk, kk > 0);
        }
        tc_commit(&ctl->s_full[x][buf]);
        tc_commit(&k_empty[s]);   // the K stage goes back to the producer when these MMAs have read it
        if (PERSISTENT && j == seen.total - 1) tc_commit(&ctl->q_empty[x]);   // the super-tile's last read of this tile's Q
      };
      auto issue_qk = [&](int j) {
        const uint32_t g = ring + (uint32_t)seen.entry(j);
        const int s = g & (kStages - 1);
        wait(&ctl->k_full[s], (g / kStages) & 1, kWaitKFull);
        if (!ok) return;
        tc_fence_after();
        if (elect_one()) qk_mmas(j, s);
        __syncwarp();
      };

      if (seen.total > 0) {
        skip_both(0, seen.entry(0));
        if (ok) wait(&ctl->q_full, q_loads & 1, kWaitQ);
        if (ok) issue_qk(0);
        if (ok && seen.total > 1) {
          skip_k(seen.entry(0) + 1, seen.entry(1));
          if (ok) issue_qk(1);
        }
      } else {
        if (PERSISTENT) {
          if (elect_one()) mbar_arrive(&ctl->q_empty[x]);   // this tile reads no Q in this super-tile
          __syncwarp();
        }
        skip_both(0, nkv);
      }
      // Per step: everything that can be checked before P arrives is (V of this step, K of the S two steps
      // ahead, the other tile's entries in between), so that nothing but the MMAs themselves stands between
      // "P(i) is in TMEM" and "S(i+2) complete" -- that span has to fit into one softmax step.
      int u_prev = -1, u = seen.total > 0 ? seen.entry(0) : -1, u1 = seen.total > 1 ? seen.entry(1) : -1;
      for (int i = 0; ok && i < seen.total; ++i) {
        const bool ahead = i + 2 < seen.total;
        const int u2 = ahead ? seen.entry(i + 2) : -1;
        // entries between consecutive ones of this tile belong to the other tile only (rare)
        if (i > 0 && u != u_prev + 1) skip_v(u_prev + 1, u);
        if (ok && ahead && u2 != u1 + 1) skip_k(u1 + 1, u2);
        if (!ok) break;
        const uint32_t gv = ring + (uint32_t)u, gk = ring + (uint32_t)(ahead ? u2 : 0);
        const int sv = gv & (kStages - 1), sk = gk & (kStages - 1);
        const uint32_t gs = sbase + (uint32_t)i, buf = gs & 1u, ppar = (gs >> 1) & 1u;
        // operands of this step's MMAs, ready before the polls: between "P has arrived" and the MMAs being
        // queued nothing should be left to compute
        const uint64_t v_desc = v_desc0 + (uint64_t)(sv * (kKBytes >> 4));
        const uint32_t sp_tmem = tmem + col_s(x, buf);
        const bool last_pv_but_one = i + 2 == seen.total;
        {
          // The TMA operands are normally there already, and so is P by the time the issuer comes back from
          // queueing the previous batch: one poll of each barrier, issued back to back, and one vote.
          const bool v_there = mbar_try_wait(&ctl->v_full[sv], (gv / kStages) & 1);
          const bool k_there = !ahead || mbar_try_wait(&ctl->k_full[sk], (gk / kStages) & 1);
          const bool p_there = mbar_try_wait(&ctl->p_full[x][buf], ppar);
          if (!__all_sync(0xffffffffu, v_there && k_there && p_there)) {
            wait(&ctl->v_full[sv], (gv / kStages) & 1, kWaitVFull);
            if (ok && ahead) wait(&ctl->k_full[sk], (gk / kStages) & 1, kWaitKFull);
            // P(i) is in TMEM (first half of its S buffer) and O has been rescaled if it had to be
            if (ok) wait(&ctl->p_full[x][buf], ppar, kWaitP);
            if (!ok) break;
          }
        }
        {
          bool got = true;
          if (elect_one()) got = pipe_acquire(ctl, p.status);
          ok = __all_sync(0xffffffffu, got);
          if (!ok) break;
        }
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < kBN / 16; ++kk) {
            // V is MN-major: 16 tokens = two 8-row groups (2048 B); dims 64-127 live kKBytes/2 further on
            tc_mma_ts(o_tmem, sp_tmem + kk * 8, v_desc + (uint64_t)(kk * (2048 >> 4)), idesc_pv, (i > 0 || kk > 0) ? 1u : 0u);
          }
          // "O is quiet" is normally read off the next S (see the softmax side); the last step has no such S
          if (last_pv_but_one) tc_commit(&ctl->pv_done[x]);
          tc_commit(&v_empty[sv]);   // the V stage goes back to the producer when these MMAs have read it
          // S(i+2) into the buffer P(i) is being read from: behind O += P(i) V(i) in this thread's order
          if (ahead) qk_mmas(i + 2, sk);
          pipe_release(ctl);
        }
        __syncwarp();
        u_prev = u;
        u = u1;
        u1 = u2;
      }
      if (ok && seen.total > 0) {
        if (elect_one()) tc_commit(&ctl->o_full[x]);
        __syncwarp();
        skip_both(seen.entry(seen.total - 1) + 1, nkv);
      }
      ring += (uint32_t)nkv;
      sbase += (uint32_t)seen.total;
      q_loads += nkv > 0 ? 1u : 0u;
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int x = warp >> 2;                              // which query tile this warpgroup owns
    const int row = tid & 127;                            // tile row == TMEM lane
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    uint32_t sbase = 0;    // S/P buffers this tile has used before this super-tile
    uint32_t n_pv = 0;     // completed phases of pv_done[x]: super-tiles in which this tile had two or more entries
    uint32_t n_o = 0;      // completed phases of o_full[x]: super-tiles in which this tile had any entry
    bool ok = true;

    for (uint32_t n = 0; ok; ++n) {
      int unit = (int)blockIdx.x;
      if (PERSISTENT) {
        const int slot = n & 1;
        ok = mbar_wait(&ctl->tile_full[slot], (n >> 1) & 1, ctl, p.status, kWaitTile);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        unit = *(volatile int*)&ctl->tile_id[slot];
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->tile_empty[slot]);
        if (unit < 0) break;
      } else if (n > 0) {
        break;
      }
      const TileWork w = (n == 0) ? w_first : tile_work(unit, p);
      const int tq = w.t0 + x;
      const TileSeen seen = tile_seen(x == 0 || w.active1, tq, w.tb, w.nb, w.local_b);
      const int64_t i_tok = (int64_t)tq * kBM + row;        // query position
      const int bi = (int)(i_tok >> 6);
      const int lo_band = bi + 1 - w.local_b;               // first band block this row sees
      const int sink_b = w.sink_b, local_b = w.local_b;

      float m_used = -INFINITY;  // max the exponentials are taken against (log2 units)
      float l = 0.f;

      for (int i = 0; i < seen.total; ++i) {
        const int jb = w.tb.block(seen.entry(i));
        const uint32_t gs = sbase + (uint32_t)i, buf = gs & 1u;
        ok = mbar_wait(&ctl->s_full[x][buf], (gs >> 1) & 1u, ctl, p.status, kWaitS);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t sv[64];
        {
          uint32_t (&lo32)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sv[0]);
          uint32_t (&hi32)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sv[32]);
          tmem_ld32(lane_base + col_s(x, buf), lo32);
          tmem_ld32(lane_base + col_s(x, buf) + 32, hi32);
          tmem_wait_ld();
        }
        const bool edge = (jb >= 2 * tq) || (jb >= sink_b && jb == 2 * tq + 1 - local_b);
        if (edge) {
          // key c of the block is visible iff the row sees the block at all, c <= query - j0 (causal) and
          // c < N - j0 (inside the sequence): one 32-bit limit per row, one compare and select per key
          const bool row_sees = (jb <= bi) && (jb < sink_b || jb >= lo_band);
          const int64_t j0 = (int64_t)jb * kBN;
          const int64_t lim64 = min(i_tok - j0, p.N - 1 - j0);
          const int limit = row_sees ? (int)max((int64_t)-1, min(lim64, (int64_t)63)) : -1;
#pragma unroll
          for (int c = 0; c < 64; ++c) {
            if (c > limit) sv[c] = 0xff800000u;  // -inf
          }
        }
        // row max of the raw scores, four independent chains of three-input max
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 64; c += 8) {
#pragma unroll
          for (int r = 0; r < 4; ++r) mx[r] = fmax3(mx[r], __uint_as_float(sv[c + 2 * r]), __uint_as_float(sv[c + 2 * r + 1]));
        }
        // scale_log2 > 0, so the max commutes with the scaling
        const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
        // lazy rescale: move the reference max only when it grew by more than 2^8
        float factor = 1.f;
        if (mt > m_used + kLazyMaxSlack) {
          factor = (m_used == -INFINITY) ? 1.f : exp2f(m_used - mt);
          m_used = mt;
        }
        const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
        uint32_t pk[32];
        // scaling, max subtraction and the row sum on packed pairs (one issue slot for two values)
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(neg_m, neg_m);
        float2 ls2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          const float2 x2 = __ffma2_rn(make_float2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), sc2, nm2);
          const float2 p2 = make_float2(exp2f(x2.x), exp2f(x2.y));
          ls2[(c >> 1) & 1] = __fadd2_rn(ls2[(c >> 1) & 1], p2);
          // P has the tensors' dtype (the MMA wants A and B in one format): with bf16 its 8-bit mantissa is the
          // largest rounding error of the bf16 path
          pk[c >> 1] = Cvt<T>::pack(p2.x, p2.y);
        }
        l = fmaf(l, factor, (ls2[0].x + ls2[0].y) + (ls2[1].x + ls2[1].y));
        // P row -> TMEM, over the first half of the S buffer it came from (two values per column, even key in
        // the low half).  The buffer's previous reader, P.V(i-2), finished before S(i) was written into it.
        tmem_st32(lane_base + col_s(x, buf), pk);
        if (i > 0 && __any_sync(0xffffffffu, factor != 1.f)) {
          // O may only be touched when P.V(i-1), the last MMA that accumulates into it, has finished.  S(i+1)
          // was issued right behind it by the same thread, so "S(i+1) complete" says so; the last step has no
          // next S and gets a commit of its own.
          ok = (i + 1 < seen.total)
                   ? mbar_wait(&ctl->s_full[x][(gs + 1) & 1u], ((gs + 1) >> 1) & 1u, ctl, p.status, kWaitS)
                   : mbar_wait(&ctl->pv_done[x], n_pv & 1u, ctl, p.status, kWaitPV);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < DH; c0 += 32) {
            uint32_t ov[32];
            tmem_ld32(lane_base + col_o(x) + c0, ov);
            tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * factor);
            tmem_st32(lane_base + col_o(x) + c0, ov);
          }
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&ctl->p_full[x][buf]);
      }
      if (!ok) break;

      if (seen.total == 0 && (x == 0 || w.active1) && i_tok < p.N) {
        // a tile that sees no key at all (no sink block and no window block): its rows are zero, like the rows
        // of a visible tile whose own mask is empty
        uint8_t* orow = reinterpret_cast<uint8_t*>(p.out) +
                        ((int64_t)w.b * p.o_sb + i_tok * p.o_sn + (int64_t)w.h * p.o_sh) * (OUT_F32 ? 4 : 2);
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll 1
        for (int c = 0; c < DH * (OUT_F32 ? 4 : 2); c += 16) *reinterpret_cast<uint4*>(orow + c) = z;
      }
      if (seen.total > 0) {
        ok = mbar_wait(&ctl->o_full[x], n_o & 1u, ctl, p.status, kWaitO);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
        // Thread r holds row r, and rows lie a whole token apart in the output: stored from here, every store
        // instruction would touch 32 lines.  Instead each warp turns its 32 rows x 128 bytes around in shared
        // memory (16-byte pieces, XOR-swizzled by the row so that neither side has bank conflicts) and stores
        // whole 128-byte lines, four rows per instruction.
        constexpr int kEs = OUT_F32 ? 4 : 2;
        constexpr int kFlushCols = 128 / kEs;               // output columns in 128 bytes
        // (the addresses are derived here, behind an opaque copy of the thread's indices, so that the compiler does
        // not keep them in registers across the step loop of the persistent form)
        int ln = lane, wp = warp;
        asm volatile("" : "+r"(ln), "+r"(wp));
        uint8_t* const stage = smem + kSmemStage + wp * kStageBytes;
        uint8_t* const mine = stage + ln * 128;
        const int sw = ln & 7, piece = ln & 7, sub = ln >> 3;
        const int64_t tok0 = (int64_t)tq * kBM + (wp & 3) * 32 + sub;   // row of this lane's first store
        uint8_t* const obase = reinterpret_cast<uint8_t*>(p.out) +
                               ((int64_t)w.b * p.o_sb + tok0 * p.o_sn + (int64_t)w.h * p.o_sh) * kEs + piece * 16;
#pragma unroll 1
        for (int c0 = 0; c0 < DH; c0 += kFlushCols) {
#pragma unroll
          for (int cc = 0; cc < kFlushCols; cc += 32) {
            uint32_t ov[32];
            tmem_ld32(lane_base + col_o(x) + c0 + cc, ov);
            tmem_wait_ld();
            if (OUT_F32) {
#pragma unroll
              for (int c = 0; c < 32; c += 4) {
                float4 f = make_float4(__uint_as_float(ov[c]) * inv_l, __uint_as_float(ov[c + 1]) * inv_l,
                                       __uint_as_float(ov[c + 2]) * inv_l, __uint_as_float(ov[c + 3]) * inv_l);
                *reinterpret_cast<float4*>(mine + (((c >> 2) ^ sw) << 4)) = f;
              }
            } else {
#pragma unroll
              for (int c = 0; c < 32; c += 8) {
                uint4 uo;
                uo.x = Cvt<T>::pack(__uint_as_float(ov[c]) * inv_l, __uint_as_float(ov[c + 1]) * inv_l);
                uo.y = Cvt<T>::pack(__uint_as_float(ov[c + 2]) * inv_l, __uint_as_float(ov[c + 3]) * inv_l);
                uo.z = Cvt<T>::pack(__uint_as_float(ov[c + 4]) * inv_l, __uint_as_float(ov[c + 5]) * inv_l);
                uo.w = Cvt<T>::pack(__uint_as_float(ov[c + 6]) * inv_l, __uint_as_float(ov[c + 7]) * inv_l);
                *reinterpret_cast<uint4*>(mine + ((((cc + c) >> 3) ^ sw) << 4)) = uo;
              }
            }
          }
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int r = it * 4 + sub;                      // row of the warp's 32
            const uint4 val = *reinterpret_cast<const uint4*>(stage + r * 128 + ((piece ^ (r & 7)) << 4));
            if (tok0 + it * 4 < p.N) *reinterpret_cast<uint4*>(obase + (int64_t)(it * 4) * p.o_sn * kEs + c0 * kEs) = val;
          }
          __syncwarp();
        }
        // the next super-tile's first O += P V overwrites O; it is issued only after every thread of this
        // tile has arrived with its first P, i.e. after these loads
        tc_fence_before();
      }
      sbase += (uint32_t)seen.total;
      n_pv += seen.total >= 2 ? 1u : 0u;
      n_o += seen.total > 0 ? 1u : 0u;
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// Self-test of the bounded wait: one thread waits, with a short limit, on a barrier nobody arrives at.
// The wait must give up, set the abort flag and leave its code in the status words; the kernel then
// returns normally and the context stays usable.
__global__ void wait_selftest_kernel(int32_t* status, long long limit_cycles) {
  __shared__ Ctl ctl;
  if (threadIdx.x == 0) {
    mbar_init(&ctl.q_full, 1);
    ctl.abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const bool ok = mbar_try_wait(&ctl.q_full, 0) || mbar_wait_slow(&ctl.q_full, 0, &ctl, status, kWaitQ, limit_cycles);
    if (ok) status[0] = -1;  // cannot happen: nothing arrives on the barrier
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess) {
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(ptr);
  return fn;
}

// (B, H, N, D) tensor with element strides (sb, sh, sn, 1) -> 4-d map (D, N, H, B), box (64, rows, 1, 1)
int make_map(CUtensorMap* map, const void* base, int dtype, int B, int H, int64_t N, int D, int64_t sb, int64_t sh,
             int64_t sn, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_error_text("prefill: cuTensorMapEncodeTiled entry point not available");
    return MOA_ERR_CUDA;
  }
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)H, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)sn * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == MOA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error_text("prefill: cuTensorMapEncodeTiled rejected the tensor (alignment or stride)");
    return MOA_ERR_INVALID_ARG;
  }
  return MOA_OK;
}

template <typename T, bool F32, int DH, bool PERSISTENT>
int launch_prefill(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PrefillParams& p,
                   dim3 grid, cudaStream_t stream) {
  auto kern = moa_prefill_kernel<T, F32, DH, PERSISTENT>;
  // The shared-memory opt-in is a per-device attribute of the function: keep the "done" flag per device
  // ordinal (one process may drive several GPUs) and per instantiation.
  constexpr int kMaxDevices = 64;
  static bool configured[kMaxDevices];
  int dev = -1;
  MOA_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices || !configured[dev]) {
    MOA_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    if (dev >= 0 && dev < kMaxDevices) configured[dev] = true;
  }
  kern<<<grid, kThreads, kSmemBytes, stream>>>(mq, mk, mv, p);
  MOA_CUDA_CHECK(cudaGetLastError());
  return MOA_OK;
}

}  // namespace
}  // namespace moa

extern "C" int moa_prefill_fwd(const void* q, const void* k, const void* v, void* out, int64_t q_sb, int64_t q_sh,
                               int64_t q_sn, int64_t k_sb, int64_t k_sh, int64_t k_sn, int64_t v_sb, int64_t v_sh,
                               int64_t v_sn, int64_t o_sb, int64_t o_sn, int64_t o_sh, const int32_t* sink_blocks,
                               const int32_t* local_blocks, int B, int H, int64_t N, int D, float sm_scale,
                               int dtype, int out_f32, int32_t* status, moa_stream_t stream) {
  using namespace moa;
  MOA_REQUIRE(q && k && v && out && sink_blocks && local_blocks && status, "prefill: null pointer");
  MOA_REQUIRE(B > 0 && H > 0 && N > 0, "prefill: bad shape");
  MOA_REQUIRE(N < (1LL << 31) - 512, "prefill: sequence too long");
  MOA_REQUIRE(sm_scale > 0.f, "prefill: sm_scale must be positive");
  if (D != 64 && D != 128) {
    set_error_text("prefill: head_dim must be 64 or 128");
    return MOA_ERR_UNSUPPORTED;
  }
  if (dtype != MOA_F16 && dtype != MOA_BF16) {
    set_error_text("prefill: dtype must be MOA_F16 or MOA_BF16");
    return MOA_ERR_UNSUPPORTED;
  }
  const int64_t strides[] = {q_sb, q_sh, q_sn, k_sb, k_sh, k_sn, v_sb, v_sh, v_sn};
  for (int64_t s : strides) MOA_REQUIRE(s > 0 && s % 8 == 0, "prefill: q/k/v strides must be positive multiples of 8 elements");
  MOA_REQUIRE(((uintptr_t)q % 16 == 0) && ((uintptr_t)k % 16 == 0) && ((uintptr_t)v % 16 == 0) &&
                  ((uintptr_t)out % 16 == 0),
              "prefill: pointers must be 16-byte aligned");
  MOA_REQUIRE(o_sb % 8 == 0 && o_sn % 8 == 0 && o_sh % 8 == 0, "prefill: out strides must be multiples of 8 elements");
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = make_map(&mq, q, dtype, B, H, N, D, q_sb, q_sh, q_sn, kBM)) != MOA_OK) return rc;
  if ((rc = make_map(&mk, k, dtype, B, H, N, D, k_sb, k_sh, k_sn, kBN)) != MOA_OK) return rc;
  if ((rc = make_map(&mv, v, dtype, B, H, N, D, v_sb, v_sh, v_sn, kBN)) != MOA_OK) return rc;
  PrefillParams p;
  p.out = out; p.o_sb = o_sb; p.o_sn = o_sn; p.o_sh = o_sh;
  p.sink_blocks = sink_blocks; p.local_blocks = local_blocks;
  p.B = B; p.H = H; p.N = N; p.scale_log2 = sm_scale * 1.4426950408889634f; p.status = status;
  const int64_t nsuper = (N + 2 * kBM - 1) / (2 * kBM);
  MOA_REQUIRE(nsuper * H * B < (1LL << 30), "prefill: too many query tiles for one launch");
  p.nsuper = (int)nsuper;
  p.num_tiles = (int)(nsuper * H * B);
  // Units are handed out in chunks of consecutive super-tiles per head (tile_coord).  Small chunks end the launch
  // on cheap tiles; large ones keep the blocks that run at the same time on few heads, whose K/V bands then stay
  // in L2 (126 MB).  Measured with 32 heads against one head after the other: 8192 tokens (134 MB of K and V)
  // chunk 2 +16 %, 16384 tokens (268 MB) chunk 4 +3 % and chunk 2 -1 %, 32768 tokens (537 MB) chunk 16 -2 %,
  // 65536 tokens chunk 16 -2 % and chunk 2 -11 %.
  const int64_t kv_bytes = (int64_t)B * H * N * D * 2 * 2;
  p.chunk = kv_bytes <= (96ll << 20) ? 1 : kv_bytes <= (192ll << 20) ? 2 : kv_bytes <= (384ll << 20) ? 4 : (int)nsuper;
  if (p.chunk > nsuper) p.chunk = (int)nsuper;
  // one block per SM (shared memory and TMEM allow no more), fewer when there are fewer super-tiles
  int sms = 0;
  {
    constexpr int kMaxDevices = 64;
    static int cached[kMaxDevices];
    int dev = -1;
    MOA_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev >= 0 && dev < kMaxDevices && cached[dev] > 0) {
      sms = cached[dev];
    } else {
      MOA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
      if (dev >= 0 && dev < kMaxDevices) cached[dev] = sms;
    }
  }
  MOA_REQUIRE(sms > 0, "prefill: no multiprocessors reported");
  // Which form: up to 16384 tokens of 32 heads (K and V up to 384 MB) the persistent one wins (4096: +8 %,
  // 16384: +5 % against one block per unit); beyond that one block per unit does (65536: +1 %), and so it does
  // when there are not even two units per SM (2048 tokens of 32 heads: +4 %; the launch then ends when the
  // heaviest unit does, whoever runs the rest).
  const bool persistent = kv_bytes <= (384ll << 20) && p.num_tiles > 2 * sms;
  dim3 grid((unsigned)(persistent && sms < p.num_tiles ? sms : p.num_tiles));
  cudaStream_t st = (cudaStream_t)stream;
  const int variant = (persistent ? 8 : 0) + (dtype == MOA_BF16 ? 4 : 0) + (out_f32 ? 2 : 0) + (D == 64 ? 1 : 0);
  switch (variant) {
    case 0: return launch_prefill<__half, false, 128, false>(mq, mk, mv, p, grid, st);
    case 1: return launch_prefill<__half, false, 64, false>(mq, mk, mv, p, grid, st);
    case 2: return launch_prefill<__half, true, 128, false>(mq, mk, mv, p, grid, st);
    case 3: return launch_prefill<__half, true, 64, false>(mq, mk, mv, p, grid, st);
    case 4: return launch_prefill<__nv_bfloat16, false, 128, false>(mq, mk, mv, p, grid, st);
    case 5: return launch_prefill<__nv_bfloat16, false, 64, false>(mq, mk, mv, p, grid, st);
    case 6: return launch_prefill<__nv_bfloat16, true, 128, false>(mq, mk, mv, p, grid, st);
    case 7: return launch_prefill<__nv_bfloat16, true, 64, false>(mq, mk, mv, p, grid, st);
    case 8: return launch_prefill<__half, false, 128, true>(mq, mk, mv, p, grid, st);
    case 9: return launch_prefill<__half, false, 64, true>(mq, mk, mv, p, grid, st);
    case 10: return launch_prefill<__half, true, 128, true>(mq, mk, mv, p, grid, st);
    case 11: return launch_prefill<__half, true, 64, true>(mq, mk, mv, p, grid, st);
    case 12: return launch_prefill<__nv_bfloat16, false, 128, true>(mq, mk, mv, p, grid, st);
    case 13: return launch_prefill<__nv_bfloat16, false, 64, true>(mq, mk, mv, p, grid, st);
    case 14: return launch_prefill<__nv_bfloat16, true, 128, true>(mq, mk, mv, p, grid, st);
    default: return launch_prefill<__nv_bfloat16, true, 64, true>(mq, mk, mv, p, grid, st);
  }
}

extern "C" int moa_selftest_bounded_wait(int32_t* status, int64_t limit_cycles, moa_stream_t stream) {
  using namespace moa;
  MOA_REQUIRE(status != nullptr, "selftest: null status");
  MOA_REQUIRE(limit_cycles > 0 && limit_cycles <= 2000000000ll, "selftest: limit must be within (0, 2e9] cycles");
  wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, (long long)limit_cycles);
  MOA_CUDA_CHECK(cudaGetLastError());
  return MOA_OK;
}
