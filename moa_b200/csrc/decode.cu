// Split-K flash-decoding over per-head ring caches, with the ring append fused in.
//
// Work decomposition: the flattened cache axis (B, S = sum of head capacities) is cut into
// fixed-size chunks of `chunk` rows; thread block (c, b) streams the rows of chunk c of batch
// row b.  Every block therefore moves the same number of bytes when the rings are full, however
// different the heads' capacities are, and no work table is needed: the block finds the head(s)
// its chunk overlaps from head_start[b, :].  For each overlapped head it produces a partial
// (max, sum, o[D]) in fp32; the last block to finish a head (atomic ticket) merges that head's
// partials, writes the output row and — in fused-append mode — advances the ring metadata.  No
// block ever waits for another one.
//
// Memory traffic per step is the algorithmic minimum (every valid K and V row once) plus
// (D+4)*4 bytes of partials per (head, chunk).
#include <stdio.h>

#include "common.cuh"

namespace moa {
namespace {

constexpr int kDecodeWarps = 4;
constexpr int kDecodeThreads = kDecodeWarps * 32;
#ifndef MOA_DECODE_TILE_ITERS
#define MOA_DECODE_TILE_ITERS 8
#endif
constexpr int kTileIters = MOA_DECODE_TILE_ITERS;  // 16-byte loads of K (and of V) in flight per thread
constexpr int kMinChunk = 128, kMaxChunk = 2048;
constexpr int kMaxOutPeers = 8;

// Rows per block when the caller passes chunk = 0.  A block pays a fixed latency chain (metadata,
// partial write, ticket) whatever it streams, so chunks should be long; and the grid should fill
// every resident-block slot of the GPU (`slots` = SMs x blocks per SM, asked from the runtime) in
// whole rounds.  Take the smallest number of rounds whose chunk (rows of one batch row / blocks per
// batch row, rounded up to 32) stays within kMaxChunk.
inline int auto_chunk_for(int B, int64_t S, int64_t slots) {
  for (int rounds = 1; rounds <= 16; ++rounds) {
    const int64_t per_row = (rounds * slots) / B > 0 ? (rounds * slots) / B : 1;
    int64_t chunk = (S + per_row - 1) / per_row;
    chunk = (chunk + 31) / 32 * 32;
    if (chunk <= kMaxChunk) return (int)(chunk < kMinChunk ? kMinChunk : chunk);
  }
  return kMaxChunk;
}
int decode_slots();  // defined after the kernel
inline int auto_chunk(int B, int64_t S) { return auto_chunk_for(B, S, decode_slots()); }

struct DecodeParams {
  const void* q;
  void* k_cache;
  void* v_cache;
  const void* k_new;
  const void* v_new;
  void* out;
  int64_t out_bs, out_hs;
  void* out_peer[kMaxOutPeers];  // further destinations of every output row (other GPUs' gather buffers)
  int n_out_peers;
  int64_t q_bs, q_hs;      // element strides of q (a row of D contiguous)
  int64_t new_bs, new_hs;  // element strides shared by k_new and v_new
  const int64_t* head_start;
  int64_t* valid_len;
  int64_t* update_index;
  int64_t* mask_cache;
  const int64_t* static_size;
  const void* rope_cos;  // (B, D) or nullptr: rotary embedding of this step applied to q and k_new in the kernel
  const void* rope_sin;
  int64_t kv_len;
  int B, H;
  int64_t S;
  float scale_log2;  // sm_scale * log2(e)
  int* tickets;      // (B, H), zero between launches; one more word behind them counts the rows written (barrier)
  float* partials;   // (B, nchunks + H, D + 4)
  // cross-GPU barrier at the end of the launch (moa_decode_gather_fwd with flags given), else bar_world == 0:
  uint32_t* bar_flags[kMaxOutPeers];  // bar_flags[g]: rank g's flag words (one per rank), mapped into this process
  int bar_rank, bar_world;
  uint32_t* bar_epoch;                // this rank's call counter in device memory
  long long bar_limit;                // bound of the wait, in SM cycles
  int32_t* bar_status;                // int32[4]: {21, rank waited for, call number, this rank} when the wait ran out
  int64_t slots_per_batch;
  int chunk;
};

__host__ __device__ inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

// Largest h with head_start[h] <= row (head_start ascending); every lane returns the result.
__device__ __forceinline__ int find_head(const int64_t* hs, int H, int64_t row, int lane) {
  int count = 0;
  for (int base = 0; base < H; base += 32) {
    const int h = base + lane;
    const bool le = (h < H) && (hs[h] <= row);
    count += __popc(__ballot_sync(0xffffffffu, le));
  }
  return count > 0 ? count - 1 : 0;
}

// Rotary embedding of the 8 dims [8*l16, 8*l16+8) of one row held by this lane:
//   x' = x*cos + rotate_half(x)*sin,  rotate_half(x)[d] = d < D/2 ? -x[d + D/2] : x[d - D/2]
// (the Llama convention).  The partner dims live in lane l16 ^ (LPR/2) of the LPR lanes that share
// the row.  Computed in fp32, rounded once to T.  `mask` names the lanes that execute the call.
template <typename T, int LPR>
__device__ __forceinline__ uint4 rope8(const uint4& x, const T* cos_row, const T* sin_row, int l16, unsigned long long mask) {
  float xf[8], cf[8], sf[8];
  unpack8<T>(x, xf);
  unpack8<T>(*reinterpret_cast<const uint4*>(cos_row + l16 * 8), cf);
  unpack8<T>(*reinterpret_cast<const uint4*>(sin_row + l16 * 8), sf);
  const bool upper = l16 >= LPR / 2;
  float r[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float partner = __shfl_xor_sync((unsigned)mask, xf[j], LPR / 2);
    r[j] = fmaf(xf[j], cf[j], (upper ? partner : -partner) * sf[j]);
  }
  uint4 o;
  o.x = Cvt<T>::pack(r[0], r[1]); o.y = Cvt<T>::pack(r[2], r[3]);
  o.z = Cvt<T>::pack(r[4], r[5]); o.w = Cvt<T>::pack(r[6], r[7]);
  return o;
}

// Element d of output row (b, h): to `out` and to every further destination (same strides).  OUT_F32 stores
// the fp32 value (the mode the bf16 path is checked in); otherwise it is rounded once to T.
template <typename T, bool OUT_F32>
__device__ __forceinline__ void store_out(const DecodeParams& p, int b, int h, int d, float o) {
  const int64_t off = (int64_t)b * p.out_bs + (int64_t)h * p.out_hs + d;
  if (OUT_F32) {
    reinterpret_cast<float*>(p.out)[off] = o;
#pragma unroll 1
    for (int g = 0; g < p.n_out_peers; ++g) reinterpret_cast<float*>(p.out_peer[g])[off] = o;
  } else {
    const T v = static_cast<T>(o);
    reinterpret_cast<T*>(p.out)[off] = v;
#pragma unroll 1
    for (int g = 0; g < p.n_out_peers; ++g) reinterpret_cast<T*>(p.out_peer[g])[off] = v;
  }
}

// Every output row of a launch is written by exactly one block.  The block that writes the last of the B*H rows
// tells every rank "this rank's rows of call n are stored" and waits (bounded) until every rank has told this
// one the same: when the kernel has finished, this rank's gather buffer holds all ranks' rows.  Called by all
// threads of a block that has written `rows_written` > 0 rows.
__device__ __noinline__ void decode_peer_barrier(const DecodeParams* pp, int rows_written) {
  const DecodeParams& p = *pp;
  __shared__ uint32_t sm_epoch;
  __shared__ int sm_is_last;
  const int tid = threadIdx.x;
  __syncthreads();                               // all of this block's row stores are issued
  if (tid == 0) {
    __threadfence_system();                      // this block's rows first
    int* rows_done = p.tickets + (int64_t)p.B * p.H;
    const int before = atomicAdd(rows_done, rows_written);
    sm_is_last = (before + rows_written == p.B * p.H);
    if (sm_is_last) {
      __threadfence_system();                    // ... and everybody else's, whose counts this thread has seen
      *rows_done = 0;                            // ready for the next launch
      const uint32_t e = *p.bar_epoch + 1u;
      *p.bar_epoch = e;
      sm_epoch = e;
    }
  }
  __syncthreads();
  if (sm_is_last && tid < p.bar_world) {
    const uint32_t epoch = sm_epoch;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.bar_flags[tid] + p.bar_rank), "r"(epoch) : "memory");
    const uint32_t* mine = p.bar_flags[p.bar_rank] + tid;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; ++spin) {
      uint32_t seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if ((int32_t)(seen - epoch) >= 0) break;
      if ((spin & 63u) == 0 && clock64() - t0 > p.bar_limit) {
        if (atomicCAS(&p.bar_status[0], 0, 21) == 0) {
          p.bar_status[1] = tid;
          p.bar_status[2] = (int32_t)epoch;
          p.bar_status[3] = p.bar_rank;
        }
        break;
      }
    }
    __threadfence_system();
  }
}

template <typename T, int D, bool OUT_F32>
__global__ void __launch_bounds__(kDecodeThreads) moa_decode_kernel(const __grid_constant__ DecodeParams p) {
  constexpr int LPR = D / 8;    // lanes that share one cache row (16 bytes each)
  constexpr int RPI = 32 / LPR; // rows a warp covers with one load instruction
  constexpr int TILE = RPI * kTileIters;
  constexpr int GROUPS = kDecodeWarps * RPI;
  constexpr int REC = D + 4;
  static_assert(D == 64 || D == 128, "head_dim");

  __shared__ float sm_m[GROUPS];
  __shared__ float sm_l[GROUPS];
  __shared__ __align__(16) float sm_acc[GROUPS][D];
  __shared__ int sm_last;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sub = lane / LPR, li = lane % LPR;
  const int b = blockIdx.y;
  const int64_t c = blockIdx.x;
  const int64_t lo = c * p.chunk;
  const int64_t hi = min(lo + (int64_t)p.chunk, p.S);
  const int64_t* hs_row = p.head_start + (int64_t)b * p.H;
  const bool fused = p.k_new != nullptr;

  const T* kc = reinterpret_cast<const T*>(p.k_cache) + (int64_t)b * p.S * D;
  const T* vc = reinterpret_cast<const T*>(p.v_cache) + (int64_t)b * p.S * D;

  // Heads without any rows (head_start[h] == head_start[h+1]) are nobody's chunk: the first block of the
  // batch row writes their (all-zero) output, so that every (b, h) row of `out` is defined.
  int rows_written = 0;   // output rows this block has written (the same in all threads)
  if (c == 0) {
    for (int h = 0; h < p.H; ++h) {
      const int64_t hs = hs_row[h];
      const int64_t he = (h + 1 < p.H) ? hs_row[h + 1] : p.S;
      if (he <= hs) {
        if (tid < D) store_out<T, OUT_F32>(p, b, h, tid, 0.f);
        ++rows_written;
      }
    }
  }

  for (int h = find_head(hs_row, p.H, lo, lane); h < p.H; ++h) {
    const int64_t hs = hs_row[h];
    if (hs >= hi) break;
    const int64_t he = (h + 1 < p.H) ? hs_row[h + 1] : p.S;
    if (he <= lo || he <= hs) continue;
    const int64_t cap = he - hs;
    const int64_t bh = (int64_t)b * p.H + h;
    const int64_t valid_pre = p.valid_len[bh];
    const int64_t upd = fused ? p.update_index[bh] : -1;
    const int64_t valid_post = fused ? valid_pre + (valid_pre < cap ? 1 : 0) : valid_pre;
    const int64_t seg_lo = max(lo, hs);
    const int64_t seg_hi = min(hi, hs + valid_post);
    const int64_t new_off = (int64_t)b * p.new_bs + (int64_t)h * p.new_hs;
    const T* knew = fused ? reinterpret_cast<const T*>(p.k_new) + new_off : nullptr;
    const T* vnew = fused ? reinterpret_cast<const T*>(p.v_new) + new_off : nullptr;

    // Fused append: the block whose chunk holds the write slot stores the new K and V rows (K with the
    // rotary embedding applied when cos/sin are given), then the whole block reads them back from the
    // cache like any other row.  No other block reads that row: it lies in this chunk only.
    const bool rope = p.rope_cos != nullptr;
    const T* cos_row = rope ? reinterpret_cast<const T*>(p.rope_cos) + (int64_t)b * D : nullptr;
    const T* sin_row = rope ? reinterpret_cast<const T*>(p.rope_sin) + (int64_t)b * D : nullptr;
    if (fused && upd >= lo && upd < hi && upd >= hs && upd < he) {   // uniform over the block
      if (warp == 0) {
        const int l16 = lane % LPR;
        if (lane < LPR) {
          uint4 ku = *reinterpret_cast<const uint4*>(knew + l16 * 8);
          if (rope) ku = rope8<T, LPR>(ku, cos_row, sin_row, l16, (1ull << LPR) - 1ull);
          *reinterpret_cast<uint4*>(const_cast<T*>(kc) + upd * D + l16 * 8) = ku;
        } else if (lane < 2 * LPR) {
          *reinterpret_cast<uint4*>(const_cast<T*>(vc) + upd * D + l16 * 8) =
              *reinterpret_cast<const uint4*>(vnew + l16 * 8);
        }
      }
      __syncthreads();
    }

    // q slice of this lane (rotated if asked), pre-scaled so that softmax runs in base 2
    float qf[8];
    {
      uint4 qu = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_bs +
                                                 (int64_t)h * p.q_hs + li * 8);
      if (rope) qu = rope8<T, LPR>(qu, cos_row, sin_row, li, 0xffffffffull);
      unpack8<T>(qu, qf);
#pragma unroll
      for (int j = 0; j < 8; ++j) qf[j] *= p.scale_log2;
    }

    float m = -INFINITY, l = 0.f;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;

    for (int64_t row0 = seg_lo + (int64_t)warp * TILE; row0 < seg_hi; row0 += (int64_t)kDecodeWarps * TILE) {
      uint4 kr[kTileIters], vr[kTileIters];
#pragma unroll
      for (int i = 0; i < kTileIters; ++i) {
        // rows past the segment re-read its last row (a valid address); their score is masked
        const int64_t r = min(row0 + i * RPI + sub, seg_hi - 1);
        kr[i] = ld_stream16(kc + r * D + li * 8);
      }
#pragma unroll
      for (int i = 0; i < kTileIters; ++i) {
        const int64_t r = min(row0 + i * RPI + sub, seg_hi - 1);
        vr[i] = ld_stream16(vc + r * D + li * 8);
      }
      float s[kTileIters];
      float mt = -INFINITY;
#pragma unroll
      for (int i = 0; i < kTileIters; ++i) {
        float kf[8];
        unpack8<T>(kr[i], kf);
        float d = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) d = fmaf(qf[j], kf[j], d);
#pragma unroll
        for (int off = LPR / 2; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
        const int64_t r = row0 + i * RPI + sub;
        s[i] = (r < seg_hi) ? d : -INFINITY;
        mt = fmaxf(mt, s[i]);
      }
      const float m_new = fmaxf(m, mt);
      if (m_new != -INFINITY) {
        const float corr = exp2f(m - m_new);  // m == -inf gives 0
        l *= corr;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] *= corr;
#pragma unroll
        for (int i = 0; i < kTileIters; ++i) {
          const float pr = exp2f(s[i] - m_new);  // masked rows give 0
          l += pr;
          float vf[8];
          unpack8<T>(vr[i], vf);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = fmaf(pr, vf[j], acc[j]);
        }
        m = m_new;
      }
    }

    // combine the GROUPS running states of this block
    const int g = warp * RPI + sub;
    if (li == 0) {
      sm_m[g] = m;
      sm_l[g] = l;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) sm_acc[g][li * 8 + j] = acc[j];
    __syncthreads();

    float M = -INFINITY;
#pragma unroll
    for (int gg = 0; gg < GROUPS; ++gg) M = fmaxf(M, sm_m[gg]);
    float L = 0.f, O = 0.f;
    if (M != -INFINITY) {
      for (int gg = 0; gg < GROUPS; ++gg) {
        const float w = exp2f(sm_m[gg] - M);
        L += sm_l[gg] * w;
        if (tid < D) O += sm_acc[gg][tid] * w;
      }
    }

    const int64_t first_chunk = hs / p.chunk;
    const int64_t nslots = (he - 1) / p.chunk - first_chunk + 1;
    bool last = true;
    if (nslots > 1) {
      float* rec = p.partials + ((int64_t)b * p.slots_per_batch + c + h) * REC;
      if (tid < D) rec[4 + tid] = O;
      if (tid == 0) {
        rec[0] = M;
        rec[1] = L;
      }
      __threadfence();
      __syncthreads();
      if (tid == 0) sm_last = (atomicAdd(&p.tickets[bh], 1) == (int)nslots - 1);
      __syncthreads();
      last = sm_last != 0;
      if (last) {
        __threadfence();
        float Mg = -INFINITY;
        for (int64_t sidx = 0; sidx < nslots; ++sidx) {
          const float* r2 = p.partials + ((int64_t)b * p.slots_per_batch + first_chunk + sidx + h) * REC;
          Mg = fmaxf(Mg, __ldcg(r2));
        }
        float Lg = 0.f, Og = 0.f;
        if (Mg != -INFINITY) {
          for (int64_t sidx = 0; sidx < nslots; ++sidx) {
            const float* r2 = p.partials + ((int64_t)b * p.slots_per_batch + first_chunk + sidx + h) * REC;
            const float w = exp2f(__ldcg(r2) - Mg);
            Lg += __ldcg(r2 + 1) * w;
            if (tid < D) Og += __ldcg(r2 + 4 + tid) * w;
          }
        }
        L = Lg;
        O = Og;
        if (tid == 0) p.tickets[bh] = 0;  // ready for the next launch
      }
    }
    if (last) {
      ++rows_written;
      if (tid < D) store_out<T, OUT_F32>(p, b, h, tid, (L > 0.f) ? O / L : 0.f);
      if (fused && tid == 0) {
        // every other block of this head has already read the old values (it took its ticket
        // after reading them), so the metadata can advance now
        p.valid_len[bh] = valid_post;
        if (p.mask_cache) p.mask_cache[(int64_t)b * p.S + upd] = 1;
        p.update_index[bh] = ring_next_index(upd, hs, cap, p.static_size[h], p.kv_len);
      }
    }
    __syncthreads();  // shared buffers are reused by the next head of this chunk
  }

  // Barrier across the GPUs, inside the launch (out of line: it runs once per block at most and must not cost
  // the streaming loop registers).
  if (p.bar_world > 0 && rows_written > 0) decode_peer_barrier(&p, rows_written);   // uniform over the block
}

// Resident-block slots of the current device for this kernel (kept per device ordinal: one process may
// drive several GPUs); 148 x 5 if no device can be asked (a build or test machine without a GPU).
constexpr int kMaxDevices = 64;
int decode_slots() {
  static int cached[kMaxDevices];   // zero-initialised; benign race: every writer stores the same value
  int dev = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    (void)cudaGetLastError();
    return 148 * 5;
  }
  if (cached[dev] > 0) return cached[dev];
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess &&
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moa_decode_kernel<__half, 128, false>, kDecodeThreads,
                                                    0) == cudaSuccess &&
      sms > 0 && per_sm > 0) {
    cached[dev] = sms * per_sm;
    return cached[dev];
  }
  (void)cudaGetLastError();
  return 148 * 5;
}

template <typename T>
int launch_decode(const DecodeParams& p, int D, bool out_f32, dim3 grid, cudaStream_t stream) {
  const int variant = (D == 64 ? 0 : D == 128 ? 2 : -1);
  switch (variant < 0 ? -1 : variant + (out_f32 ? 1 : 0)) {
    case 0: moa_decode_kernel<T, 64, false><<<grid, kDecodeThreads, 0, stream>>>(p); break;
    case 1: moa_decode_kernel<T, 64, true><<<grid, kDecodeThreads, 0, stream>>>(p); break;
    case 2: moa_decode_kernel<T, 128, false><<<grid, kDecodeThreads, 0, stream>>>(p); break;
    case 3: moa_decode_kernel<T, 128, true><<<grid, kDecodeThreads, 0, stream>>>(p); break;
    default: set_error_text("decode: head_dim must be 64 or 128"); return MOA_ERR_UNSUPPORTED;
  }
  MOA_CUDA_CHECK(cudaGetLastError());
  return MOA_OK;
}

struct WsLayout {
  int64_t ticket_bytes, nchunks, slots_per_batch, total;
};
inline WsLayout ws_layout(int B, int H, int D, int64_t S, int chunk) {
  WsLayout w;
  w.ticket_bytes = round_up((int64_t)B * H * 4 + 4, 256);   // tickets + the rows-written counter of the barrier
  w.nchunks = (S + chunk - 1) / chunk;
  w.slots_per_batch = w.nchunks + H;
  w.total = w.ticket_bytes + (int64_t)B * w.slots_per_batch * (D + 4) * 4;
  return w;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// What every decode entry point passes on (the C ABI spells these out as plain arguments).
struct DecodeCall {
  const void* q; void* k_cache; void* v_cache; const void* k_new; const void* v_new; void* out;
  int64_t q_bs, q_hs, new_bs, new_hs, out_bs, out_hs;
  const int64_t* head_start; int64_t* valid_len; int64_t* update_index; int64_t* mask_cache;
  const int64_t* static_size; int64_t kv_len;
  int B, H, D; int64_t S; float sm_scale; int dtype, out_f32;
  void* workspace; int64_t workspace_bytes; int chunk; cudaStream_t stream;
  const void* rope_cos; const void* rope_sin;
  void* const* out_peers; int n_out_peers;
  void* const* bar_flags; int bar_rank, bar_world; uint32_t* bar_epoch; int64_t bar_limit; int32_t* bar_status;
};

// Validates the arguments, lays out the workspace and launches the kernel.
int decode_launch_with_scratch(const DecodeCall& a) {
  MOA_REQUIRE(a.q && a.k_cache && a.v_cache && a.out && a.head_start && a.valid_len, "decode: null pointer");
  MOA_REQUIRE((a.k_new == nullptr) == (a.v_new == nullptr), "decode: k_new and v_new must both be given or both be NULL");
  MOA_REQUIRE(a.B > 0 && a.H > 0 && a.S > 0 && a.B <= 65535, "decode: bad shape");
  if (a.k_new) MOA_REQUIRE(a.update_index && a.static_size, "decode: fused append needs update_index and static_size");
  MOA_REQUIRE((a.rope_cos == nullptr) == (a.rope_sin == nullptr), "decode: rope_cos and rope_sin go together");
  MOA_REQUIRE(a.rope_cos == nullptr || a.k_new != nullptr, "decode: the rotary embedding is applied in the fused-append mode only");
  MOA_REQUIRE(aligned16(a.q) && a.q_bs % 8 == 0 && a.q_hs % 8 == 0 && a.q_bs >= 0 && a.q_hs >= 0,
              "decode: q must be 16-byte aligned with strides that are multiples of 8 elements");
  if (a.k_new)
    MOA_REQUIRE(aligned16(a.k_new) && aligned16(a.v_new) && a.new_bs % 8 == 0 && a.new_hs % 8 == 0 && a.new_bs >= 0 &&
                    a.new_hs >= 0,
                "decode: k_new/v_new must be 16-byte aligned with strides that are multiples of 8 elements");
  MOA_REQUIRE(aligned16(a.k_cache) && aligned16(a.v_cache), "decode: the caches must be 16-byte aligned");
  MOA_REQUIRE(a.n_out_peers >= 0 && a.n_out_peers <= kMaxOutPeers && (a.n_out_peers == 0 || a.out_peers != nullptr),
              "decode: at most 8 further output destinations");
  int chunk = a.chunk;
  if (chunk <= 0) chunk = auto_chunk(a.B, a.S);
  const WsLayout w = ws_layout(a.B, a.H, a.D, a.S, chunk);
  if (!a.workspace || a.workspace_bytes < w.total) {
    set_error_text("decode: workspace missing or smaller than moa_decode_workspace_bytes()");
    return MOA_ERR_WORKSPACE;
  }
  MOA_REQUIRE(w.nchunks <= 2147483647LL, "decode: too many chunks");
  DecodeParams p;
  p.q = a.q; p.k_cache = a.k_cache; p.v_cache = a.v_cache; p.k_new = a.k_new; p.v_new = a.v_new; p.out = a.out;
  p.out_bs = a.out_bs; p.out_hs = a.out_hs; p.q_bs = a.q_bs; p.q_hs = a.q_hs; p.new_bs = a.new_bs; p.new_hs = a.new_hs;
  p.n_out_peers = a.n_out_peers;
  for (int g = 0; g < kMaxOutPeers; ++g) p.out_peer[g] = g < a.n_out_peers ? a.out_peers[g] : nullptr;
  for (int g = 0; g < a.n_out_peers; ++g) MOA_REQUIRE(p.out_peer[g] != nullptr, "decode: null output destination");
  p.head_start = a.head_start; p.valid_len = a.valid_len;
  p.update_index = a.update_index; p.mask_cache = a.mask_cache; p.static_size = a.static_size; p.kv_len = a.kv_len;
  p.rope_cos = a.rope_cos; p.rope_sin = a.rope_sin;
  p.bar_world = 0; p.bar_rank = 0; p.bar_epoch = nullptr; p.bar_limit = 0; p.bar_status = nullptr;
  for (int g = 0; g < kMaxOutPeers; ++g) p.bar_flags[g] = nullptr;
  if (a.bar_flags != nullptr) {
    MOA_REQUIRE(a.bar_world >= 1 && a.bar_world <= kMaxOutPeers && a.bar_rank >= 0 && a.bar_rank < a.bar_world,
                "decode_gather: the barrier serves 1..8 ranks");
    MOA_REQUIRE(a.bar_epoch != nullptr && a.bar_status != nullptr, "decode_gather: the barrier needs its call counter and status words");
    MOA_REQUIRE(a.bar_limit > 0 && a.bar_limit <= 20000000000ll, "decode_gather: barrier limit must be within (0, 2e10] cycles");
    for (int g = 0; g < a.bar_world; ++g) {
      MOA_REQUIRE(a.bar_flags[g] != nullptr, "decode_gather: null flag pointer");
      p.bar_flags[g] = reinterpret_cast<uint32_t*>(a.bar_flags[g]);
    }
    p.bar_world = a.bar_world; p.bar_rank = a.bar_rank; p.bar_epoch = a.bar_epoch; p.bar_limit = (long long)a.bar_limit;
    p.bar_status = a.bar_status;
  }
  p.B = a.B; p.H = a.H; p.S = a.S; p.scale_log2 = a.sm_scale * 1.4426950408889634f;
  p.tickets = reinterpret_cast<int*>(a.workspace);
  p.partials = reinterpret_cast<float*>(reinterpret_cast<char*>(a.workspace) + w.ticket_bytes);
  p.slots_per_batch = w.slots_per_batch; p.chunk = chunk;
  dim3 grid((unsigned)w.nchunks, (unsigned)a.B);
  if (a.dtype == MOA_F16) return launch_decode<__half>(p, a.D, a.out_f32 != 0, grid, a.stream);
  if (a.dtype == MOA_BF16) return launch_decode<__nv_bfloat16>(p, a.D, a.out_f32 != 0, grid, a.stream);
  set_error_text("decode: dtype must be MOA_F16 or MOA_BF16");
  return MOA_ERR_UNSUPPORTED;
}

}  // namespace moa

// The argument list shared by the decode entry points, in the order of include/moa_b200.h.
#define MOA_DECODE_ARGS_DECL                                                                                       \
  const void *q, void *k_cache, void *v_cache, const void *k_new, const void *v_new, void *out,                    \
      int64_t q_batch_stride, int64_t q_head_stride, int64_t new_batch_stride, int64_t new_head_stride,            \
      int64_t out_batch_stride, int64_t out_head_stride, const int64_t *head_start, int64_t *valid_len,            \
      int64_t *update_index, int64_t *mask_cache, const int64_t *static_size, int64_t kv_len, int B, int H, int D, \
      int64_t S, float sm_scale, int dtype, int out_f32

static moa::DecodeCall make_call(MOA_DECODE_ARGS_DECL, void* workspace, int64_t workspace_bytes, int chunk,
                                 moa_stream_t stream) {
  moa::DecodeCall a;
  a.q = q; a.k_cache = k_cache; a.v_cache = v_cache; a.k_new = k_new; a.v_new = v_new; a.out = out;
  a.q_bs = q_batch_stride; a.q_hs = q_head_stride; a.new_bs = new_batch_stride; a.new_hs = new_head_stride;
  a.out_bs = out_batch_stride; a.out_hs = out_head_stride;
  a.head_start = head_start; a.valid_len = valid_len; a.update_index = update_index; a.mask_cache = mask_cache;
  a.static_size = static_size; a.kv_len = kv_len; a.B = B; a.H = H; a.D = D; a.S = S; a.sm_scale = sm_scale;
  a.dtype = dtype; a.out_f32 = out_f32; a.workspace = workspace; a.workspace_bytes = workspace_bytes; a.chunk = chunk;
  a.stream = (cudaStream_t)stream; a.rope_cos = nullptr; a.rope_sin = nullptr; a.out_peers = nullptr; a.n_out_peers = 0;
  a.bar_flags = nullptr; a.bar_rank = 0; a.bar_world = 0; a.bar_epoch = nullptr; a.bar_limit = 0; a.bar_status = nullptr;
  return a;
}
#define MOA_DECODE_ARGS_PASS                                                                                     \
  q, k_cache, v_cache, k_new, v_new, out, q_batch_stride, q_head_stride, new_batch_stride, new_head_stride,      \
      out_batch_stride, out_head_stride, head_start, valid_len, update_index, mask_cache, static_size, kv_len, B, \
      H, D, S, sm_scale, dtype, out_f32

extern "C" {

int64_t moa_decode_workspace_bytes(int B, int H, int D, int64_t S, int chunk) {
  if (B <= 0 || H <= 0 || D <= 0 || S <= 0) return 0;
  if (chunk <= 0) chunk = moa::auto_chunk(B, S);
  return moa::ws_layout(B, H, D, S, chunk).total;
}

int moa_decode_workspace_init(void* workspace, int64_t workspace_bytes, moa_stream_t stream) {
  MOA_REQUIRE(workspace && workspace_bytes > 0, "workspace_init: null workspace");
  MOA_CUDA_CHECK(cudaMemsetAsync(workspace, 0, (size_t)workspace_bytes, (cudaStream_t)stream));
  return MOA_OK;
}

int moa_decode_fwd(MOA_DECODE_ARGS_DECL, void* workspace, int64_t workspace_bytes, int chunk, moa_stream_t stream) {
  return moa::decode_launch_with_scratch(make_call(MOA_DECODE_ARGS_PASS, workspace, workspace_bytes, chunk, stream));
}

int moa_decode_rope_fwd(MOA_DECODE_ARGS_DECL, const void* rope_cos, const void* rope_sin, void* workspace,
                        int64_t workspace_bytes, int chunk, moa_stream_t stream) {
  MOA_REQUIRE(rope_cos && rope_sin && k_new && v_new, "decode_rope: needs k_new, v_new, rope_cos and rope_sin");
  moa::DecodeCall a = make_call(MOA_DECODE_ARGS_PASS, workspace, workspace_bytes, chunk, stream);
  a.rope_cos = rope_cos;
  a.rope_sin = rope_sin;
  return moa::decode_launch_with_scratch(a);
}

int moa_decode_gather_fwd(MOA_DECODE_ARGS_DECL, const void* rope_cos, const void* rope_sin, void* const* out_peers,
                          int n_out_peers, void* const* barrier_flags, int rank, int world, uint32_t* epoch_counter,
                          int64_t limit_cycles, int32_t* barrier_status, void* workspace, int64_t workspace_bytes,
                          int chunk, moa_stream_t stream) {
  MOA_REQUIRE((rope_cos == nullptr) == (rope_sin == nullptr), "decode_gather: rope_cos and rope_sin go together");
  moa::DecodeCall a = make_call(MOA_DECODE_ARGS_PASS, workspace, workspace_bytes, chunk, stream);
  a.rope_cos = rope_cos;
  a.rope_sin = rope_sin;
  a.out_peers = out_peers;
  a.n_out_peers = n_out_peers;
  a.bar_flags = barrier_flags;
  a.bar_rank = rank; a.bar_world = world; a.bar_epoch = epoch_counter; a.bar_limit = limit_cycles;
  a.bar_status = barrier_status;
  return moa::decode_launch_with_scratch(a);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Decode entry point that brings its own scratch (no workspace argument, no allocation).
//
// Some hosts of this library cannot hand the decode step a workspace: an inference server that has
// already given every free byte of HBM to its KV-cache pool, a plugin running inside someone else's
// step loop where cudaMalloc (and the device-wide synchronisation it implies) is not acceptable,
// or a thin FFI binding without an allocator of its own.  For them the tickets and split partials
// live in the fixed device array below, which every GPU that loads the library holds until the
// process exits.
// ------------------------------------------------------------------------------------------------
#include <mutex>

namespace moa {
namespace {

static __device__ __align__(256) unsigned char g_decode_scratch[MOA_DECODE_STATIC_SCRATCH_BYTES];

void* g_decode_scratch_addr[kMaxDevices];  // device address of g_decode_scratch, per device ordinal
std::mutex g_decode_scratch_mutex;

// In host code `g_decode_scratch` is only a handle for the symbol, not an address a kernel can use;
// the address on the current device comes from cudaGetSymbolAddress.  Looked up once per device.
int decode_static_scratch(void** ptr) {
  int dev = -1;
  MOA_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    set_error_text("decode_static: device ordinal out of range");
    return MOA_ERR_INVALID_ARG;
  }
  std::lock_guard<std::mutex> lock(g_decode_scratch_mutex);
  if (g_decode_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    MOA_CUDA_CHECK(cudaGetSymbolAddress(&p, g_decode_scratch));
    g_decode_scratch_addr[dev] = p;
  }
  *ptr = g_decode_scratch_addr[dev];
  return MOA_OK;
}

}  // namespace
}  // namespace moa

extern "C" int moa_decode_fwd_static(MOA_DECODE_ARGS_DECL, int chunk, moa_stream_t stream) {
  using namespace moa;
  MOA_REQUIRE(B > 0 && H > 0 && D > 0 && S > 0, "decode_static: bad shape");
  if (chunk <= 0) chunk = auto_chunk(B, S);
  const WsLayout w = ws_layout(B, H, D, S, chunk);
  if (w.total > (int64_t)MOA_DECODE_STATIC_SCRATCH_BYTES) {
    char msg[256];
    snprintf(msg, sizeof(msg),
             "decode_static: this shape needs %lld bytes of scratch, the built-in array holds %lld; "
             "use moa_decode_fwd with a caller-provided workspace",
             (long long)w.total, (long long)MOA_DECODE_STATIC_SCRATCH_BYTES);
    set_error_text(msg);
    return MOA_ERR_TOO_LARGE;
  }
  void* scratch = nullptr;
  const int rc = decode_static_scratch(&scratch);
  if (rc != MOA_OK) return rc;
  // The array keeps whatever the previous call left; the tickets must start at zero.
  MOA_CUDA_CHECK(cudaMemsetAsync(scratch, 0, (size_t)w.ticket_bytes, (cudaStream_t)stream));
  return decode_launch_with_scratch(
      make_call(MOA_DECODE_ARGS_PASS, scratch, MOA_DECODE_STATIC_SCRATCH_BYTES, chunk, stream));
}
