/*
 * moa_b200 — C ABI of the B200 (sm_100a) kernels for MoA's attention hot path.
 *
 * Every entry point takes plain device pointers and sizes, enqueues its work on the CUDA
 * stream it is given, never synchronises the device and never allocates device memory
 * (the moa_peer_alloc / moa_peer_free pair is the one exception, and says so).
 * The return value is a moa_status (0 = MOA_OK); moa_strerror() names it and
 * moa_last_error_detail() gives the CUDA error text of the calling thread's last failure.
 *
 * The comment on each function names the part of thu-nics/MoA it stands in for
 * (paths relative to that repository).
 */
#ifndef MOA_B200_H_
#define MOA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOA_ABI_VERSION 2

typedef void* moa_stream_t; /* a cudaStream_t; NULL is the legacy default stream */

enum moa_dtype { MOA_F16 = 0, MOA_BF16 = 1 };

enum moa_status {
  MOA_OK = 0,
  MOA_ERR_INVALID_ARG = 1,  /* null pointer, bad shape or stride                         */
  MOA_ERR_UNSUPPORTED = 2,  /* head_dim or dtype the kernels are not built for            */
  MOA_ERR_CUDA = 3,         /* a CUDA runtime/driver call failed; see moa_last_error_detail */
  MOA_ERR_WORKSPACE = 4,    /* workspace missing or too small                            */
  MOA_ERR_DEVICE_WAIT = 5,  /* a bounded wait inside a kernel ran out (reported via status word) */
  MOA_ERR_TOO_LARGE = 6     /* size beyond a fixed limit of the entry point              */
};

int moa_abi_version(void);
const char* moa_strerror(int status);
const char* moa_last_error_detail(void);

/* ------------------------------------------------------------------------------------------
 * Decode: flash-decoding over the per-head ring caches of one layer.
 *
 * Replaces the external `flashinfer.moa_decode(q, k, v, head_start_index, head_valid_length,
 * sm_scale)` call at MoA/kernels/mixture_of_attention.py:465-473 and, when k_new/v_new are
 * given, also the decode branch of StaticCircularCache.update
 * (MoA/attention/cache_utils.py:1020-1058) in the same launch.
 *
 *   q            (B, H, D)   element (b, h, d) at q[b*q_batch_stride + h*q_head_stride + d]: the reference's
 *                            (B,H,1,D) and (B,1,H,D) are q_batch_stride = H*D, q_head_stride = D; a slice of a
 *                            fused QKV projection output (B, 3*H*D) is q_batch_stride = 3*H*D.  Rows must be
 *                            16-byte aligned (pointer aligned, strides multiples of 8 elements)
 *   k_cache,
 *   v_cache      (B, S, D)   contiguous, S = sum of per-head capacities; head h owns rows
 *                            [head_start[b,h], head_start[b,h+1]) (last head: up to S)
 *   k_new, v_new (B, H, D)   with the element strides (new_batch_stride, new_head_stride), shared by both.
 *                            Both NULL: attention only over the first valid_len[b,h] rows of
 *                            each head.  Both non-NULL: fused append — the new row is written at
 *                            update_index[b,h], attention runs over the rows that are valid
 *                            after the append (the new token is attended), and afterwards
 *                            valid_len, update_index and mask_cache are advanced exactly as
 *                            cache_utils.py:1031-1054 does (kv_len is the layer's _kv_len
 *                            before this step; static_size is static_cache_size[layer]).
 *   out          element (b, h, d) is written at out[b*out_batch_stride + h*out_head_stride + d]
 *                            so (B,1,H,D) and a slice of a wider gather buffer are both possible.
 *                            A head that owns no rows at all gets zeros.
 *   out_f32      non-zero: out is float32 (same math, the fp32 result stored unrounded) — the mode the
 *                            bf16 path is checked in; zero: out has the dtype of q
 *   head_start,
 *   valid_len,
 *   update_index (B, H) int64;  mask_cache (B, S) int64 or NULL;  static_size (H) int64
 *   workspace    moa_decode_workspace_bytes() bytes, zeroed once by
 *                moa_decode_workspace_init(); reusable by later calls on the same stream.
 *                Two launches that overlap in time must not share a workspace.
 *   chunk        rows of the flattened cache per thread block; 0 lets the library choose
 *                (128..2048 by problem size).  moa_decode_workspace_bytes must be asked with
 *                the same chunk value that is passed here.
 * ------------------------------------------------------------------------------------------ */
int64_t moa_decode_workspace_bytes(int B, int H, int D, int64_t S, int chunk);
int moa_decode_workspace_init(void* workspace, int64_t workspace_bytes, moa_stream_t stream);
int moa_decode_fwd(const void* q, void* k_cache, void* v_cache, const void* k_new, const void* v_new, void* out,
                   int64_t q_batch_stride, int64_t q_head_stride, int64_t new_batch_stride,
                   int64_t new_head_stride, int64_t out_batch_stride, int64_t out_head_stride,
                   const int64_t* head_start, int64_t* valid_len, int64_t* update_index,
                   int64_t* mask_cache, const int64_t* static_size, int64_t kv_len,
                   int B, int H, int D, int64_t S, float sm_scale, int dtype, int out_f32,
                   void* workspace, int64_t workspace_bytes, int chunk, moa_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * moa_decode_rope_fwd: the fused-append decode step with the rotary embedding folded in.
 * Stands for the decode-time sequence of LlamaMixtureAttention.forward
 * (MoA/models/llama/modeling_llama.py:234-326): split of the projection output -> apply_rotary_pos_emb(q, k)
 * -> cache.update -> attention, in one launch.  q and k_new are the raw projection outputs (through their
 * strides they may be slices of one fused QKV output); rope_cos / rope_sin are this step's (B, D) tables in
 * the tensors' dtype (the position_embeddings the model computes once per forward, Llama rotate_half
 * convention).  The rotated K row is what is stored in the cache.
 * Everything else as moa_decode_fwd with k_new/v_new given.
 * ------------------------------------------------------------------------------------------ */
int moa_decode_rope_fwd(const void* q, void* k_cache, void* v_cache, const void* k_new, const void* v_new, void* out,
                        int64_t q_batch_stride, int64_t q_head_stride, int64_t new_batch_stride,
                        int64_t new_head_stride, int64_t out_batch_stride, int64_t out_head_stride,
                        const int64_t* head_start, int64_t* valid_len, int64_t* update_index,
                        int64_t* mask_cache, const int64_t* static_size, int64_t kv_len,
                        int B, int H, int D, int64_t S, float sm_scale, int dtype, int out_f32,
                        const void* rope_cos, const void* rope_sin,
                        void* workspace, int64_t workspace_bytes, int chunk, moa_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * moa_decode_gather_fwd: the decode step of a head shard that delivers its output rows to every GPU of
 * the node, and waits for the other GPUs' rows, in the same launch.  Stands for the attention of
 * LlamaMixtureAttention.forward (MoA/models/llama/modeling_llama.py:315-326) on one rank plus the gather of
 * the ranks' head shards into (B, 1, H, D) that has to precede o_proj (:329-330) when heads are sharded; the
 * reference itself is single-GPU and has no such step.
 *   out_peers    host array of n_out_peers (0..8) device pointers: the same place (out plus this rank's head
 *                offset) in the other GPUs' gather buffers, mapped into this process (moa_peer_open).  Every
 *                output row is stored to out and, with the same strides, to each of them (plain stores over
 *                NVLink; nothing is loaded from a peer).
 *   rope_cos/sin both NULL or both given (as moa_decode_rope_fwd).
 *   barrier_flags, rank, world, epoch_counter, limit_cycles, barrier_status
 *                the cross-rank barrier at the end of the launch, with the meaning they have in
 *                moa_peer_barrier (flags: host array of `world` device pointers; epoch_counter: a device uint32
 *                of this rank, zero at the start, required here): the block that writes the last output row of
 *                the launch publishes the call number to every rank and waits, for at most limit_cycles, until
 *                every rank has published it to this one.  When the kernel has finished, this rank's buffer
 *                holds all ranks' rows of the call (or barrier_status says which rank did not arrive).
 *                barrier_flags NULL: the launch only stores; the caller orders the peers' reads itself
 *                (moa_peer_barrier after it).  The workspace is the one of moa_decode_fwd.
 * Everything else as moa_decode_fwd.
 * ------------------------------------------------------------------------------------------ */
int moa_decode_gather_fwd(const void* q, void* k_cache, void* v_cache, const void* k_new, const void* v_new,
                          void* out, int64_t q_batch_stride, int64_t q_head_stride, int64_t new_batch_stride,
                          int64_t new_head_stride, int64_t out_batch_stride, int64_t out_head_stride,
                          const int64_t* head_start, int64_t* valid_len, int64_t* update_index,
                          int64_t* mask_cache, const int64_t* static_size, int64_t kv_len,
                          int B, int H, int D, int64_t S, float sm_scale, int dtype, int out_f32,
                          const void* rope_cos, const void* rope_sin, void* const* out_peers, int n_out_peers,
                          void* const* barrier_flags, int rank, int world, uint32_t* epoch_counter,
                          int64_t limit_cycles, int32_t* barrier_status,
                          void* workspace, int64_t workspace_bytes, int chunk, moa_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * moa_decode_fwd_static: moa_decode_fwd without the workspace argument.  It has no counterpart
 * in the reference; it exists for hosts that cannot allocate device memory on the decode path
 * (a server whose KV-cache pool already owns all free HBM, a plugin that must not trigger
 * cudaMalloc's device-wide synchronisation, an FFI binding with no allocator).  The scratch is
 * a fixed device array of MOA_DECODE_STATIC_SCRATCH_BYTES inside the library, held by every
 * GPU that loads it until the process exits.  The call allocates nothing.
 *   - Shapes whose scratch need (moa_decode_workspace_bytes) exceeds the array are refused
 *     with MOA_ERR_TOO_LARGE; config 1 (B16 H32 D128, 67k slots per row) needs 4.7 MB.
 *   - The first call on each device looks up the array's device address (once, with that device
 *     current); make that first call before any stream capture.
 *   - All calls on a device share the one array: calls that can overlap on the GPU (different
 *     streams, or concurrent host threads) race on it.  Serialise them or use moa_decode_fwd.
 * Arguments and semantics otherwise as moa_decode_fwd.
 * ------------------------------------------------------------------------------------------ */
#define MOA_DECODE_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
int moa_decode_fwd_static(const void* q, void* k_cache, void* v_cache, const void* k_new, const void* v_new,
                          void* out, int64_t q_batch_stride, int64_t q_head_stride, int64_t new_batch_stride,
                          int64_t new_head_stride, int64_t out_batch_stride, int64_t out_head_stride,
                          const int64_t* head_start, int64_t* valid_len, int64_t* update_index,
                          int64_t* mask_cache, const int64_t* static_size, int64_t kv_len,
                          int B, int H, int D, int64_t S, float sm_scale, int dtype, int out_f32,
                          int chunk, moa_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Ring-cache bookkeeping (StaticCircularCache.update, MoA/attention/cache_utils.py:953-1164).
 *
 * moa_cache_append: decode branch (:1020-1058) without attention.  k_new/v_new (B,H,D) with
 *   element strides nk_b, nk_h (row of D contiguous); NULL k_new/v_new = the reference's
 *   update_cache_content=False (indices, lengths and mask advance, payload untouched).
 *
 * moa_cache_scan_mask: for the prefill branch with an attention mask (:1062-1086).
 *   mask (B, N) int64 with row stride mask_stride; writes pos (B, N) int32 = position of the
 *   j-th unmasked token of the row, and count (B) int32 = number of unmasked tokens.
 *
 * moa_cache_fill: prefill branch (:1060-1164).  k, v (B,H,N,D) with element strides
 *   (sb, sh, sn; D contiguous).  pos/count from moa_cache_scan_mask, or both NULL for "no
 *   mask".  Keeps a token iff it is among the last circ_h unmasked tokens or its slot lies
 *   in the static part (:1122-1133); advances valid_len (+= kept), update_index (:1110) and
 *   mask_cache (:1149).  max_cap = largest per-head capacity (sizes the grid).
 * ------------------------------------------------------------------------------------------ */
int moa_cache_append(void* k_cache, void* v_cache, const void* k_new, const void* v_new,
                     int64_t new_batch_stride, int64_t new_head_stride,
                     const int64_t* head_start, int64_t* valid_len, int64_t* update_index,
                     int64_t* mask_cache, const int64_t* static_size, int64_t kv_len,
                     int B, int H, int D, int64_t S, int dtype, moa_stream_t stream);
int moa_cache_scan_mask(const int64_t* mask, int64_t mask_stride, int32_t* pos, int32_t* count,
                        int B, int64_t N, moa_stream_t stream);
int moa_cache_fill(const void* k, const void* v, int64_t sb, int64_t sh, int64_t sn,
                   void* k_cache, void* v_cache, const int32_t* pos, const int32_t* count,
                   const int64_t* head_start, int64_t* valid_len, int64_t* update_index,
                   int64_t* mask_cache, const int64_t* static_size, int64_t kv_len,
                   int B, int H, int64_t N, int D, int64_t S, int64_t max_cap, int dtype,
                   moa_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Prefill: causal sink + sliding-window block-sparse attention.
 *
 * Replaces `flashinfer.moa_prefill(q, k, v, causal=True, num_global_blocks, num_band_blocks,
 * kv_layout="HND")` (MoA/kernels/mixture_of_attention.py:435-444) and the Triton kernel
 * `_sparse_attention_prefill_moa_fwd_kernel` (MoA/kernels/block_sparse_attention_prefill.py:
 * 473-696): q-block bi (64 rows) sees kv-block j iff j <= bi and (j < sink_blocks[h] or
 * j >= bi + 1 - local_blocks[h]); inside a block the mask is causal.
 *
 *   q, k, v  (B, H, N, D), D = 64 or 128, with element strides (sb, sh, sn), D contiguous,
 *            every stride a multiple of 8 elements, base pointers 16-byte aligned
 *   out      written as out[b*ob + n*on + h*oh + d]; (B,N,H,D) contiguous is ob=N*H*D, on=H*D, oh=D
 *   sink_blocks, local_blocks (H) int32 device arrays, in 64-token blocks
 *   status   device int32[8], zero on entry, owned by this launch until it has finished (launches that can
 *            overlap in time need a buffer each).  Words 0-3 report a bounded wait that gave up: a non-zero
 *            word 0 after the kernel finished means MOA_ERR_DEVICE_WAIT and out is invalid.
 *            status[0] = what was waited for (1 Q tiles, 2 a K tile, 3 a free K stage, 4 S from the
 *            tensor core, 5 P from the softmax warps, 6 the last but one P.V, 7 the final O, 8 a V
 *            tile, 9 a free V stage, 11 the issuer's turn on the tensor core, 12 the next unit of work,
 *            13 a free slot to publish it in, 14 the Q tiles to be free); status[1] = blockIdx.x,
 *            status[2] = 0, status[3] = threadIdx.x of the waiter.  Words 4-5 are the work scheduler's
 *            (next query tile to hand out, blocks finished); the kernel leaves them zero again.
 *   out_f32 non-zero: out is float32 (same math, fp32 store) — used to check the bf16 path
 * ------------------------------------------------------------------------------------------ */
int moa_prefill_fwd(const void* q, const void* k, const void* v, void* out,
                    int64_t q_sb, int64_t q_sh, int64_t q_sn,
                    int64_t k_sb, int64_t k_sh, int64_t k_sn,
                    int64_t v_sb, int64_t v_sh, int64_t v_sn,
                    int64_t o_sb, int64_t o_sn, int64_t o_sh,
                    const int32_t* sink_blocks, const int32_t* local_blocks,
                    int B, int H, int64_t N, int D, float sm_scale, int dtype, int out_f32,
                    int32_t* status, moa_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * moa_rope_qk: rotary embedding of q and k in place, one pass over both.  Replaces
 * apply_rotary_pos_emb(query_states, key_states, cos, sin) at MoA/models/llama/modeling_llama.py:252
 * for the prefill (the decode step applies it inside moa_decode_rope_fwd).
 *   q, k      (B, H, N, D) sharing the element strides (sb, sh, sn), D contiguous
 *   cos, sin  (B, N, D) tables in the tensors' dtype, element strides (cos_batch_stride, cos_token_stride);
 *             a batch stride of 0 shares one table among the batch rows
 * ------------------------------------------------------------------------------------------ */
int moa_rope_qk(void* q, void* k, int64_t sb, int64_t sh, int64_t sn, const void* cos, const void* sin,
                int64_t cos_batch_stride, int64_t cos_token_stride, int B, int H, int64_t N, int D, int dtype,
                moa_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Buffers that the GPUs of one node write into directly (what moa_decode_gather_fwd's out_peers point at),
 * and a barrier across the ranks.  No counterpart in the reference, which runs on one GPU; together with
 * moa_decode_gather_fwd they replace the all-gather of the head shards' outputs that has to precede
 * o_proj (MoA/models/llama/modeling_llama.py:329-330) when heads are sharded over GPUs.
 *
 * moa_peer_alloc / moa_peer_free: device memory of the current device that other processes can map
 *   (cudaMalloc'ed, zero-filled; these two calls allocate and free and synchronise like cudaMalloc/cudaFree:
 *   set-up time only).
 * moa_peer_export: writes the MOA_PEER_HANDLE_BYTES-byte handle of such a buffer; send it to the other ranks
 *   by any host channel.  moa_peer_open maps a handle received from another process of the same node into
 *   this process (peer access is enabled as needed) and returns the device pointer; moa_peer_close unmaps it.
 * moa_peer_barrier: enqueues a one-block kernel that (1) publishes `epoch` in word `rank` of every rank's
 *   flag array and (2) waits until all `world` words of this rank's own array have reached `epoch`.
 *   flags: host array of `world` device pointers, flags[g] = rank g's array of `world` uint32 words (zero at
 *   the start; flags[rank] is this rank's own).  Every rank calls it with the same epoch, which must grow by
 *   one from call to call; with epoch_counter given (a device uint32 of this rank, zero at the start) the
 *   kernel counts the calls itself — it uses ++*epoch_counter and ignores `epoch` — so that the launch can be
 *   captured in a CUDA graph and replayed.  Work enqueued before the barrier on this stream (stores into the peers' buffers)
 *   is visible to what the other ranks enqueue after theirs.  The wait gives up after limit_cycles SM cycles
 *   (at most 2e10): status (device int32[4], zero on entry) then holds {21, the rank waited for, epoch, rank}
 *   and the kernel returns normally.
 * ------------------------------------------------------------------------------------------ */
#define MOA_PEER_HANDLE_BYTES 64
int moa_peer_alloc(void** ptr, int64_t bytes);
int moa_peer_free(void* ptr);
int moa_peer_export(void* ptr, void* handle);
int moa_peer_open(const void* handle, void** ptr);
int moa_peer_close(void* ptr);
int moa_peer_barrier(void* const* flags, int rank, int world, uint32_t epoch, uint32_t* epoch_counter,
                     int64_t limit_cycles, int32_t* status, moa_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * moa_selftest_bounded_wait: failure-detection self-test (no counterpart in the reference, which has
 * no device-side waits).  Launches one thread that waits, for at most limit_cycles SM cycles, on an
 * mbarrier nobody arrives at, through the same bounded-wait routine the prefill kernel uses.  After
 * the kernel status[0] holds the wait code (non-zero) and status[1..3] the block/thread that gave up;
 * the kernel returns normally.  status: device int32[4], zero on entry.
 * ------------------------------------------------------------------------------------------ */
int moa_selftest_bounded_wait(int32_t* status, int64_t limit_cycles, moa_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MOA_B200_H_ */
