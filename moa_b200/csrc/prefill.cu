// Block-sparse causal prefill (attention sink + per-head sliding window) on tcgen05 / TMEM / TMA.
//
// One thread block computes one 128-row query tile of one (batch, head).  Roles:
//   warps 0-3  softmax: thread r owns query row r (= TMEM lane r); reads S from TMEM, writes
//              P (fp16/bf16) to shared memory in the 128-byte-swizzled K-major layout, keeps the
//              running max / sum, rescales O in TMEM when the max moved, runs the epilogue
//   warp  4    TMA producer (one lane): Q once, then K/V tiles of 64 tokens through a ring of
//              kStages shared-memory stages
//   warp  5    MMA issuer (one lane) and owner of the TMEM allocation:
//              S_j = Q K_j^T (M128 N64 K128) into one of two S buffers, O += P_j V_j (M128 N128 K64)
// Only the 64-token KV blocks inside "sink U band" of the tile are ever loaded; blocks outside
// are skipped, and only the (at most three) edge blocks of a tile get an element mask.
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

constexpr int kD = 128;            // head_dim this kernel is built for
constexpr int kBM = 128;           // query rows per tile
constexpr int kBN = 64;            // KV tokens per tile (= the mask's block size)
constexpr int kStages = 4;         // K/V ring depth
constexpr int kSoftmaxThreads = 128;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 256;  // O: [0,128)  S0: [128,192)  S1: [192,256)
constexpr uint32_t kColO = 0, kColS = 128;

constexpr int kQBytes = kBM * kD * 2;       // 32 KiB  (two 16 KiB halves: dims 0-63, 64-127)
constexpr int kKBytes = kBN * kD * 2;       // 16 KiB  (two 8 KiB halves)
constexpr int kStageBytes = 2 * kKBytes;    // K then V
constexpr int kPBytes = kBM * kBN * 2;      // 16 KiB
constexpr int kSmemQ = 0;
constexpr int kSmemKV = kSmemQ + kQBytes;
constexpr int kSmemP = kSmemKV + kStages * kStageBytes;
constexpr int kSmemCtl = kSmemP + 2 * kPBytes;
constexpr int kSmemBytes = kSmemCtl + 256 + 1024;  // control block + slack for 1024-byte alignment

constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s: far above any legitimate wait

// status codes written to status[0] when a wait gives up
enum { kWaitQ = 1, kWaitKVFull = 2, kWaitKVEmpty = 3, kWaitS = 4, kWaitP = 5, kWaitPV = 6, kWaitO = 7 };

struct Ctl {
  uint64_t q_full;
  uint64_t kv_full[kStages];
  uint64_t kv_empty[kStages];
  uint64_t s_full[2];
  uint64_t p_full[2];
  uint64_t pv_done;
  uint64_t o_full;
  uint32_t tmem_base;
  int abort;
};

struct PrefillParams {
  void* out;
  int64_t o_sb, o_sn, o_sh;
  const int32_t* sink_blocks;
  const int32_t* local_blocks;
  int B, H;
  int64_t N;
  float scale_log2;
  int32_t* status;
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
__device__ __noinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Ctl* ctl, int32_t* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 1023u) == 0) {
      if (*(volatile int*)&ctl->abort) return false;
      if (globaltimer_ns() - t0 > kWaitLimitNs) {
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

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

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

// Instruction descriptor for kind::f16 with fp32 accumulation.
__host__ __device__ constexpr uint32_t make_idesc(int is_bf16, int b_mn_major, int M, int N) {
  return (1u << 4) | ((uint32_t)is_bf16 << 7) | ((uint32_t)is_bf16 << 10) | ((uint32_t)b_mn_major << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// KV blocks a query tile visits: [0, nA) (sink part) then [bB, bB + nB) (band part).
struct TileBlocks {
  int nA, bB, nB;
  __device__ __forceinline__ int count() const { return nA + nB; }
  __device__ __forceinline__ int block(int i) const { return i < nA ? i : bB + (i - nA); }
};
__device__ __forceinline__ TileBlocks tile_blocks(int t, int nb, int sink_b, int local_b) {
  const int hi = min(2 * t + 2, nb);                 // blocks [0, hi) are at or below the diagonal
  TileBlocks r;
  r.nA = max(0, min(sink_b, hi));
  r.bB = max(r.nA, 2 * t + 1 - local_b);              // first band block of the upper half
  r.nB = max(0, hi - r.bB);
  return r;
}

template <typename T, bool OUT_F32>
__global__ void __launch_bounds__(kThreads, 1)
moa_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const PrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  Ctl* ctl = reinterpret_cast<Ctl*>(smem + kSmemCtl);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ntiles = (int)((p.N + kBM - 1) / kBM);
  const int t = ntiles - 1 - (int)blockIdx.x;  // heaviest tiles are scheduled first
  const int h = blockIdx.y, b = blockIdx.z;
  const int nb = (int)((p.N + kBN - 1) / kBN);
  const int sink_b = p.sink_blocks[h], local_b = p.local_blocks[h];
  const TileBlocks tb = tile_blocks(t, nb, sink_b, local_b);
  const int ntile_kv = tb.count();
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;

  if (tid == 0) {
    mbar_init(&ctl->q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&ctl->kv_full[s], 1);
      mbar_init(&ctl->kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ctl->s_full[s], 1);
      mbar_init(&ctl->p_full[s], kSoftmaxThreads);
    }
    mbar_init(&ctl->pv_done, 1);
    mbar_init(&ctl->o_full, 1);
    ctl->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *(volatile uint32_t*)&ctl->tmem_base;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(&ctl->q_full, kQBytes);
      tma_load_4d(smem + kSmemQ, &map_q, &ctl->q_full, 0, t * kBM, h, b);
      tma_load_4d(smem + kSmemQ + kQBytes / 2, &map_q, &ctl->q_full, 64, t * kBM, h, b);
      int issued = 0;
      for (int j = 0; j < ntile_kv; ++j) {
        const int s = j % kStages;
        if (!mbar_wait(&ctl->kv_empty[s], ((j / kStages) & 1) ^ 1, ctl, p.status, kWaitKVEmpty)) break;
        uint8_t* st = smem + kSmemKV + s * kStageBytes;
        const int row = tb.block(j) * kBN;
        mbar_expect_tx(&ctl->kv_full[s], kStageBytes);
        tma_load_4d(st, &map_k, &ctl->kv_full[s], 0, row, h, b);
        tma_load_4d(st + kKBytes / 2, &map_k, &ctl->kv_full[s], 64, row, h, b);
        tma_load_4d(st + kKBytes, &map_v, &ctl->kv_full[s], 0, row, h, b);
        tma_load_4d(st + kKBytes + kKBytes / 2, &map_v, &ctl->kv_full[s], 64, row, h, b);
        issued = j + 1;
      }
      if (*(volatile int*)&ctl->abort) {
        // drain: shared memory must not be released while bulk copies into it are in flight
        const uint64_t t0 = globaltimer_ns();
        for (int j = max(0, issued - kStages); j < issued; ++j) {
          while (!mbar_try_wait(&ctl->kv_full[j % kStages], (j / kStages) & 1) &&
                 globaltimer_ns() - t0 < kWaitLimitNs) {
          }
        }
        while (!mbar_try_wait(&ctl->q_full, 0) && globaltimer_ns() - t0 < kWaitLimitNs) {
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(kBf16, 0, kBM, kBN);
      constexpr uint32_t idesc_pv = make_idesc(kBf16, 1, kBM, kD);
      const uint32_t q_addr = smem_u32(smem + kSmemQ);
      bool ok = mbar_wait(&ctl->q_full, 0, ctl, p.status, kWaitQ);
      tc_fence_after();

      auto issue_qk = [&](int j) -> bool {
        const int s = j % kStages;
        if (!mbar_wait(&ctl->kv_full[s], (j / kStages) & 1, ctl, p.status, kWaitKVFull)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + kSmemKV + s * kStageBytes);
        const uint32_t d_tmem = tmem + kColS + (uint32_t)(j & 1) * kBN;
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t half = kk >> 2, off = (kk & 3) * 32;
          const uint64_t a = make_desc(q_addr + half * (kQBytes / 2) + off, 16, 1024);
          const uint64_t bd = make_desc(k_addr + half * (kKBytes / 2) + off, 16, 1024);
          tc_mma_ss(d_tmem, a, bd, idesc_qk, kk > 0);
        }
        tc_commit(&ctl->s_full[j & 1]);
        return true;
      };

      if (ok && ntile_kv > 0) ok = issue_qk(0);
      if (ok && ntile_kv > 1) ok = issue_qk(1);
      for (int j = 0; ok && j < ntile_kv; ++j) {
        if (!mbar_wait(&ctl->p_full[j & 1], (j >> 1) & 1, ctl, p.status, kWaitP)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const int s = j % kStages;
        const uint32_t v_addr = smem_u32(smem + kSmemKV + s * kStageBytes + kKBytes);
        const uint32_t p_addr = smem_u32(smem + kSmemP + (j & 1) * kPBytes);
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk) {
          const uint64_t a = make_desc(p_addr + kk * 32, 16, 1024);
          // V is MN-major: 16 tokens = two 8-row groups (2048 B); dims 64-127 live kKBytes/2 further on
          const uint64_t bd = make_desc(v_addr + kk * 2048, kKBytes / 2, 1024);
          tc_mma_ss(tmem + kColO, a, bd, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&ctl->kv_empty[s]);
        tc_commit(&ctl->pv_done);
        if (j + 2 < ntile_kv) ok = issue_qk(j + 2);
      }
      if (ok) tc_commit(&ctl->o_full);
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int row = tid;                                  // tile row == TMEM lane
    const int64_t i_tok = (int64_t)t * kBM + row;         // query position
    const int bi = (int)(i_tok >> 6);
    const int lo_band = bi + 1 - local_b;                 // first band block this row sees
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    uint8_t* p_row_base = smem + kSmemP + row * 128;
    const int sw = row & 7;

    float m_used = -INFINITY;  // max the exponentials are taken against (log2 units)
    float l = 0.f;
    bool ok = true;

    for (int j = 0; j < ntile_kv; ++j) {
      ok = mbar_wait(&ctl->s_full[j & 1], (j >> 1) & 1, ctl, p.status, kWaitS);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[64];
      {
        uint32_t (&lo32)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sv[0]);
        uint32_t (&hi32)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sv[32]);
        tmem_ld32(lane_base + kColS + (uint32_t)(j & 1) * kBN, lo32);
        tmem_ld32(lane_base + kColS + (uint32_t)(j & 1) * kBN + 32, hi32);
        tmem_wait_ld();
      }
      const int jb = tb.block(j);
      const bool edge = (jb >= 2 * t) || (jb >= sink_b && jb == 2 * t + 1 - local_b);
      float mt = -INFINITY;
      if (edge) {
        const bool row_sees = (jb <= bi) && (jb < sink_b || jb >= lo_band);
        const int64_t j0 = (int64_t)jb * kBN;
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const bool vis = row_sees && (j0 + c <= i_tok) && (j0 + c < p.N);
          const float x = vis ? __uint_as_float(sv[c]) * p.scale_log2 : -INFINITY;
          sv[c] = __float_as_uint(x);
          mt = fmaxf(mt, x);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const float x = __uint_as_float(sv[c]) * p.scale_log2;
          sv[c] = __float_as_uint(x);
          mt = fmaxf(mt, x);
        }
      }
      // lazy rescale: move the reference max only when it grew by more than 2^8
      float factor = 1.f;
      if (mt > m_used + 8.f) {
        factor = (m_used == -INFINITY) ? 1.f : exp2f(m_used - mt);
        l *= factor;
        m_used = mt;
      }
      const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        const float p0 = exp2f(__uint_as_float(sv[c]) - m_sub);
        const float p1 = exp2f(__uint_as_float(sv[c + 1]) - m_sub);
        l += p0 + p1;
        pk[c >> 1] = Cvt<T>::pack(p0, p1);
      }
      // P row -> shared memory, K-major with the 128-byte swizzle (16-byte chunk c at c ^ (row % 8))
      uint8_t* prow = p_row_base + (j & 1) * kPBytes;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        *reinterpret_cast<uint4*>(prow + ((c ^ sw) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      }
      fence_async_smem();
      // O may only be touched (and P[j&1] of two tiles ago is only free) once PV of tile j-1 is done
      if (j > 0) {
        ok = mbar_wait(&ctl->pv_done, (j - 1) & 1, ctl, p.status, kWaitPV);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, factor != 1.f)) {
#pragma unroll 1
          for (int c0 = 0; c0 < kD; c0 += 32) {
            uint32_t ov[32];
            tmem_ld32(lane_base + kColO + c0, ov);
            tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * factor);
            tmem_st32(lane_base + kColO + c0, ov);
          }
          tmem_wait_st();
        }
      }
      tc_fence_before();
      mbar_arrive(&ctl->p_full[j & 1]);
    }

    if (ok && ntile_kv > 0) {
      ok = mbar_wait(&ctl->o_full, 0, ctl, p.status, kWaitO);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && ntile_kv > 0) {
      tc_fence_after();
      const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
      const bool store = i_tok < p.N;
      uint8_t* orow = reinterpret_cast<uint8_t*>(p.out) +
                      ((int64_t)b * p.o_sb + i_tok * p.o_sn + (int64_t)h * p.o_sh) * (OUT_F32 ? 4 : 2);
#pragma unroll 1
      for (int c0 = 0; c0 < kD; c0 += 32) {
        uint32_t ov[32];
        tmem_ld32(lane_base + kColO + c0, ov);
        tmem_wait_ld();
        if (store) {
          if (OUT_F32) {
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
              float4 f = make_float4(__uint_as_float(ov[c]) * inv_l, __uint_as_float(ov[c + 1]) * inv_l,
                                     __uint_as_float(ov[c + 2]) * inv_l, __uint_as_float(ov[c + 3]) * inv_l);
              *reinterpret_cast<float4*>(orow + (c0 + c) * 4) = f;
            }
          } else {
#pragma unroll
            for (int c = 0; c < 32; c += 8) {
              uint4 u;
              u.x = Cvt<T>::pack(__uint_as_float(ov[c]) * inv_l, __uint_as_float(ov[c + 1]) * inv_l);
              u.y = Cvt<T>::pack(__uint_as_float(ov[c + 2]) * inv_l, __uint_as_float(ov[c + 3]) * inv_l);
              u.z = Cvt<T>::pack(__uint_as_float(ov[c + 4]) * inv_l, __uint_as_float(ov[c + 5]) * inv_l);
              u.w = Cvt<T>::pack(__uint_as_float(ov[c + 6]) * inv_l, __uint_as_float(ov[c + 7]) * inv_l);
              *reinterpret_cast<uint4*>(orow + (c0 + c) * 2) = u;
            }
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
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
int make_map(CUtensorMap* map, const void* base, int dtype, int B, int H, int64_t N, int64_t sb, int64_t sh,
             int64_t sn, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_error_text("prefill: cuTensorMapEncodeTiled entry point not available");
    return MOA_ERR_CUDA;
  }
  const cuuint64_t dims[4] = {(cuuint64_t)kD, (cuuint64_t)N, (cuuint64_t)H, (cuuint64_t)B};
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

template <typename T, bool F32>
int launch_prefill(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PrefillParams& p,
                   dim3 grid, cudaStream_t stream) {
  auto kern = moa_prefill_kernel<T, F32>;
  static bool configured = false;  // per instantiation
  if (!configured) {
    MOA_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    configured = true;
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
  MOA_REQUIRE(B > 0 && H > 0 && N > 0 && B <= 65535 && H <= 65535, "prefill: bad shape");
  MOA_REQUIRE(N < (1LL << 31) - 256, "prefill: sequence too long");
  if (D != kD) {
    set_error_text("prefill: head_dim must be 128");
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
  if ((rc = make_map(&mq, q, dtype, B, H, N, q_sb, q_sh, q_sn, kBM)) != MOA_OK) return rc;
  if ((rc = make_map(&mk, k, dtype, B, H, N, k_sb, k_sh, k_sn, kBN)) != MOA_OK) return rc;
  if ((rc = make_map(&mv, v, dtype, B, H, N, v_sb, v_sh, v_sn, kBN)) != MOA_OK) return rc;
  PrefillParams p;
  p.out = out; p.o_sb = o_sb; p.o_sn = o_sn; p.o_sh = o_sh;
  p.sink_blocks = sink_blocks; p.local_blocks = local_blocks;
  p.B = B; p.H = H; p.N = N; p.scale_log2 = sm_scale * 1.4426950408889634f; p.status = status;
  const int ntiles = (int)((N + kBM - 1) / kBM);
  dim3 grid((unsigned)ntiles, (unsigned)H, (unsigned)B);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == MOA_F16) {
    return out_f32 ? launch_prefill<__half, true>(mq, mk, mv, p, grid, st)
                   : launch_prefill<__half, false>(mq, mk, mv, p, grid, st);
  }
  return out_f32 ? launch_prefill<__nv_bfloat16, true>(mq, mk, mv, p, grid, st)
                 : launch_prefill<__nv_bfloat16, false>(mq, mk, mv, p, grid, st);
}
