// Ring-cache bookkeeping on the device: decode append, mask scan and prefill fill.
//
// Layout (one layer): k_cache/v_cache (B, S, D) with S = sum of per-head capacities; head h owns
// rows [head_start[b,h], head_start[b,h+1]); its first static_size[h] rows are the sink part and
// the rest is the ring.  All index tensors are int64, the types the reference's Python keeps.
#include "common.cuh"

namespace moa {
namespace {

constexpr int kFillRows = 64;      // kept tokens handled by one block of the fill kernel
constexpr int kFillThreads = 256;
constexpr int kScanThreads = 1024;

// ---- decode-branch update without attention (cache_utils.py:1020-1058) -----------------------
template <int D>
__global__ void __launch_bounds__(32) cache_append_kernel(uint16_t* k_cache, uint16_t* v_cache, const uint16_t* k_new,
                                                          const uint16_t* v_new, int64_t nbs, int64_t nhs,
                                                          const int64_t* head_start, int64_t* valid_len,
                                                          int64_t* update_index, int64_t* mask_cache,
                                                          const int64_t* static_size, int64_t kv_len, int H,
                                                          int64_t S) {
  constexpr int LPR = D / 8;
  const int h = blockIdx.x, b = blockIdx.y, lane = threadIdx.x;
  const int64_t bh = (int64_t)b * H + h;
  const int64_t hs = head_start[bh];
  const int64_t he = (h + 1 < H) ? head_start[bh + 1] : S;
  const int64_t upd = update_index[bh];
  const int64_t valid = valid_len[bh];
  __syncwarp();
  if (k_new != nullptr && upd >= 0 && upd < S) {
    for (int e = lane; e < 2 * LPR; e += 32) {
      const bool is_v = e >= LPR;
      const int l16 = e % LPR;
      const uint16_t* src = (is_v ? v_new : k_new) + (int64_t)b * nbs + (int64_t)h * nhs + l16 * 8;
      uint16_t* dst = (is_v ? v_cache : k_cache) + ((int64_t)b * S + upd) * D + l16 * 8;
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
    }
  }
  if (lane == 0) {
    if (mask_cache && upd >= 0 && upd < S) mask_cache[(int64_t)b * S + upd] = 1;
    valid_len[bh] = valid + (valid < he - hs ? 1 : 0);
    update_index[bh] = ring_next_index(upd, hs, he - hs, static_size[h], kv_len);
  }
}

// ---- attention-mask scan (cache_utils.py:1075-1086) ------------------------------------------
// pos[b, j] = position of the j-th token of row b whose mask is 1; count[b] = how many there are.
__global__ void __launch_bounds__(kScanThreads) cache_scan_mask_kernel(const int64_t* mask, int64_t mask_stride,
                                                                       int32_t* pos, int32_t* count, int64_t N) {
  __shared__ int warp_sums[kScanThreads / 32];
  __shared__ int running;
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) running = 0;
  __syncthreads();
  for (int64_t t0 = 0; t0 < N; t0 += kScanThreads) {
    const int64_t t = t0 + tid;
    const int keep = (t < N) && (mask[(int64_t)b * mask_stride + t] == 1);
    int incl = keep;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += n;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int ws = warp_sums[lane];
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, ws, off);
        if (lane >= off) ws += n;
      }
      warp_sums[lane] = ws;  // inclusive over warps
    }
    __syncthreads();
    const int base = running + (warp > 0 ? warp_sums[warp - 1] : 0);
    if (keep) pos[(int64_t)b * N + base + incl - 1] = (int32_t)t;
    __syncthreads();
    if (tid == 0) running += warp_sums[kScanThreads / 32 - 1];
    __syncthreads();
  }
  if (tid == 0) count[b] = running;
}

// ---- prefill-branch update (cache_utils.py:1060-1164) ----------------------------------------
// For head (b, h) with n unmasked tokens, ordinal j (0-based among unmasked tokens) goes to
//   idx(j) = (kv_len + j > static) ? (upd0 + j - cs) mod circ + cs : upd0 + j          (:1088-1107)
// and is kept iff  n - j <= circ  or  idx(j) < cs                                      (:1122-1133)
// The ring formula never gives idx < cs, so the kept set is a prefix [0, nB) (static formula,
// slot below cs) joined with the suffix [n - circ, n).
struct FillHead {
  int64_t hs, cap, cs, circ, upd0, stat, n, nB, a_start, kept;
};
__device__ __forceinline__ FillHead fill_head(const int64_t* head_start, const int64_t* update_index,
                                              const int64_t* static_size, const int32_t* count, int64_t kv_len,
                                              int b, int h, int H, int64_t N, int64_t S) {
  FillHead f;
  const int64_t bh = (int64_t)b * H + h;
  f.hs = head_start[bh];
  const int64_t he = (h + 1 < H) ? head_start[bh + 1] : S;
  f.cap = he - f.hs;
  f.stat = static_size[h];
  f.cs = f.hs + f.stat;
  f.circ = f.cap - f.stat;
  f.upd0 = update_index[bh];
  f.n = count ? (int64_t)count[b] : N;
  int64_t nB = min(f.stat - kv_len + 1, f.cs - f.upd0);
  f.nB = max((int64_t)0, min(nB, f.n));
  f.a_start = max(max((int64_t)0, f.n - f.circ), f.nB);
  f.kept = f.nB + (f.n - f.a_start);
  return f;
}
__device__ __forceinline__ int64_t fill_slot(const FillHead& f, int64_t kv_len, int64_t j) {
  if (kv_len + j > f.stat && f.circ > 0) return pymod(f.upd0 + j - f.cs, f.circ) + f.cs;
  return f.upd0 + j;
}

template <int D>
__global__ void __launch_bounds__(kFillThreads) cache_fill_kernel(const uint16_t* k, const uint16_t* v, int64_t sb,
                                                                  int64_t sh, int64_t sn, uint16_t* k_cache,
                                                                  uint16_t* v_cache, const int32_t* pos,
                                                                  const int32_t* count, const int64_t* head_start,
                                                                  const int64_t* update_index, int64_t* mask_cache,
                                                                  const int64_t* static_size, int64_t kv_len, int H,
                                                                  int64_t N, int64_t S) {
  constexpr int LPR = D / 8;
  constexpr int RPW = 32 / (2 * LPR) > 0 ? 32 / (2 * LPR) : 1;  // rows (K and V) a warp copies at once
  const int h = blockIdx.y, b = blockIdx.z;
  const FillHead f = fill_head(head_start, update_index, static_size, count, kv_len, b, h, H, N, S);
  const int64_t k0 = (int64_t)blockIdx.x * kFillRows;
  if (k0 >= f.kept) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / (2 * LPR), e = lane % (2 * LPR);
  const bool is_v = e >= LPR;
  const int l16 = e % LPR;
  const int64_t k_hi = min(k0 + kFillRows, f.kept);
  for (int64_t kk = k0 + warp * RPW + sub; kk < k_hi; kk += (kFillThreads / 32) * RPW) {
    if (sub >= RPW) break;
    const int64_t j = kk < f.nB ? kk : f.a_start + (kk - f.nB);
    const int64_t t = pos ? (int64_t)pos[(int64_t)b * N + j] : j;
    const int64_t idx = fill_slot(f, kv_len, j);
    if (idx < 0 || idx >= S) continue;
    const uint16_t* src = (is_v ? v : k) + (int64_t)b * sb + (int64_t)h * sh + t * sn + l16 * 8;
    uint16_t* dst = (is_v ? v_cache : k_cache) + ((int64_t)b * S + idx) * D + l16 * 8;
    *reinterpret_cast<uint4*>(dst) = ld_stream16(src);
    if (e == 0 && mask_cache) mask_cache[(int64_t)b * S + idx] = 1;
  }
}

// Runs after the copy kernel (stream order), so no copy block can see the advanced values.
__global__ void cache_fill_finalize_kernel(const int32_t* count, const int64_t* head_start, int64_t* valid_len,
                                           int64_t* update_index, const int64_t* static_size, int64_t kv_len, int B,
                                           int H, int64_t N, int64_t S) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)B * H) return;
  const int b = (int)(i / H), h = (int)(i % H);
  const FillHead f = fill_head(head_start, update_index, static_size, count, kv_len, b, h, H, N, S);
  valid_len[i] += f.kept;
  update_index[i] = fill_slot(f, kv_len, f.n);  // cache_utils.py:1110
}

// ---- rotary embedding of q and k in place (modeling_llama.py:252) -----------------------------
// One thread rotates 8 dims of the lower half of a row together with their partners in the upper half:
//   x'[d] = x[d] cos[d] - x[d + D/2] sin[d],   x'[d + D/2] = x[d + D/2] cos[d + D/2] + x[d] sin[d + D/2]
// (Llama rotate_half convention), fp32 arithmetic, one rounding.  Rows are (b, h, n); q and k share
// the (b, n) tables.
template <typename T, int D>
__global__ void __launch_bounds__(256) rope_qk_kernel(T* q, T* k, int64_t sb, int64_t sh, int64_t sn, const T* cos_t,
                                                      const T* sin_t, int64_t cs_b, int64_t cs_n, int H, int64_t N,
                                                      int64_t total) {
  constexpr int TPR = D / 16;  // threads per row
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t rowi = idx / TPR;
  if (rowi >= total) return;
  const int part = (int)(idx % TPR);
  const int64_t n = rowi % N, bh = rowi / N;
  const int h = (int)(bh % H);
  const int64_t b = bh / H;
  const T* cr = cos_t + b * cs_b + n * cs_n;
  const T* sr = sin_t + b * cs_b + n * cs_n;
  float c_lo[8], c_hi[8], s_lo[8], s_hi[8];
  unpack8<T>(*reinterpret_cast<const uint4*>(cr + part * 8), c_lo);
  unpack8<T>(*reinterpret_cast<const uint4*>(cr + D / 2 + part * 8), c_hi);
  unpack8<T>(*reinterpret_cast<const uint4*>(sr + part * 8), s_lo);
  unpack8<T>(*reinterpret_cast<const uint4*>(sr + D / 2 + part * 8), s_hi);
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    T* row = (which == 0 ? q : k) + b * sb + (int64_t)h * sh + n * sn;
    float lo[8], hi[8], olo[8], ohi[8];
    unpack8<T>(*reinterpret_cast<const uint4*>(row + part * 8), lo);
    unpack8<T>(*reinterpret_cast<const uint4*>(row + D / 2 + part * 8), hi);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      olo[j] = fmaf(lo[j], c_lo[j], -hi[j] * s_lo[j]);
      ohi[j] = fmaf(hi[j], c_hi[j], lo[j] * s_hi[j]);
    }
    uint4 a, c;
    a.x = Cvt<T>::pack(olo[0], olo[1]); a.y = Cvt<T>::pack(olo[2], olo[3]);
    a.z = Cvt<T>::pack(olo[4], olo[5]); a.w = Cvt<T>::pack(olo[6], olo[7]);
    c.x = Cvt<T>::pack(ohi[0], ohi[1]); c.y = Cvt<T>::pack(ohi[2], ohi[3]);
    c.z = Cvt<T>::pack(ohi[4], ohi[5]); c.w = Cvt<T>::pack(ohi[6], ohi[7]);
    *reinterpret_cast<uint4*>(row + part * 8) = a;
    *reinterpret_cast<uint4*>(row + D / 2 + part * 8) = c;
  }
}

template <typename T>
int launch_rope(void* q, void* k, int64_t sb, int64_t sh, int64_t sn, const void* cos_t, const void* sin_t,
                int64_t cs_b, int64_t cs_n, int B, int H, int64_t N, int D, cudaStream_t st) {
  const int64_t total = (int64_t)B * H * N;
  if (D == 128) {
    const int64_t threads = total * 8;
    rope_qk_kernel<T, 128><<<(unsigned)ceil_div64(threads, 256), 256, 0, st>>>((T*)q, (T*)k, sb, sh, sn, (const T*)cos_t,
                                                                             (const T*)sin_t, cs_b, cs_n, H, N, total);
  } else if (D == 64) {
    const int64_t threads = total * 4;
    rope_qk_kernel<T, 64><<<(unsigned)ceil_div64(threads, 256), 256, 0, st>>>((T*)q, (T*)k, sb, sh, sn, (const T*)cos_t,
                                                                            (const T*)sin_t, cs_b, cs_n, H, N, total);
  } else {
    set_error_text("rope_qk: head_dim must be 64 or 128");
    return MOA_ERR_UNSUPPORTED;
  }
  MOA_CUDA_CHECK(cudaGetLastError());
  return MOA_OK;
}

}  // namespace
}  // namespace moa

extern "C" {

int moa_rope_qk(void* q, void* k, int64_t sb, int64_t sh, int64_t sn, const void* cos_t, const void* sin_t,
                int64_t cos_batch_stride, int64_t cos_token_stride, int B, int H, int64_t N, int D, int dtype,
                moa_stream_t stream) {
  using namespace moa;
  MOA_REQUIRE(q && k && cos_t && sin_t, "rope_qk: null pointer");
  MOA_REQUIRE(B > 0 && H > 0 && N > 0, "rope_qk: bad shape");
  MOA_REQUIRE(sb % 8 == 0 && sh % 8 == 0 && sn % 8 == 0 && cos_batch_stride % 8 == 0 && cos_token_stride % 8 == 0,
              "rope_qk: strides must be multiples of 8 elements");
  MOA_REQUIRE((int64_t)B * H * N < (1ll << 40), "rope_qk: too many rows");
  if (dtype == MOA_F16)
    return launch_rope<__half>(q, k, sb, sh, sn, cos_t, sin_t, cos_batch_stride, cos_token_stride, B, H, N, D,
                               (cudaStream_t)stream);
  if (dtype == MOA_BF16)
    return launch_rope<__nv_bfloat16>(q, k, sb, sh, sn, cos_t, sin_t, cos_batch_stride, cos_token_stride, B, H, N, D,
                                      (cudaStream_t)stream);
  set_error_text("rope_qk: dtype must be MOA_F16 or MOA_BF16");
  return MOA_ERR_UNSUPPORTED;
}

int moa_cache_append(void* k_cache, void* v_cache, const void* k_new, const void* v_new, int64_t new_batch_stride,
                     int64_t new_head_stride, const int64_t* head_start, int64_t* valid_len, int64_t* update_index,
                     int64_t* mask_cache, const int64_t* static_size, int64_t kv_len, int B, int H, int D, int64_t S,
                     int dtype, moa_stream_t stream) {
  using namespace moa;
  MOA_REQUIRE(head_start && valid_len && update_index && static_size, "cache_append: null index pointer");
  MOA_REQUIRE((k_new == nullptr) == (v_new == nullptr), "cache_append: k_new and v_new go together");
  MOA_REQUIRE(k_new == nullptr || (k_cache && v_cache), "cache_append: null cache pointer");
  MOA_REQUIRE(B > 0 && H > 0 && S > 0 && B <= 65535, "cache_append: bad shape");
  MOA_REQUIRE(new_batch_stride % 8 == 0 && new_head_stride % 8 == 0, "cache_append: strides must be multiples of 8");
  MOA_REQUIRE(dtype == MOA_F16 || dtype == MOA_BF16, "cache_append: bad dtype");
  dim3 grid((unsigned)H, (unsigned)B);
  auto kc = (uint16_t*)k_cache; auto vc = (uint16_t*)v_cache;
  auto kn = (const uint16_t*)k_new; auto vn = (const uint16_t*)v_new;
  cudaStream_t st = (cudaStream_t)stream;
  if (D == 128) {
    cache_append_kernel<128><<<grid, 32, 0, st>>>(kc, vc, kn, vn, new_batch_stride, new_head_stride, head_start,
                                                  valid_len, update_index, mask_cache, static_size, kv_len, H, S);
  } else if (D == 64) {
    cache_append_kernel<64><<<grid, 32, 0, st>>>(kc, vc, kn, vn, new_batch_stride, new_head_stride, head_start,
                                                 valid_len, update_index, mask_cache, static_size, kv_len, H, S);
  } else {
    set_error_text("cache_append: head_dim must be 64 or 128");
    return MOA_ERR_UNSUPPORTED;
  }
  MOA_CUDA_CHECK(cudaGetLastError());
  return MOA_OK;
}

int moa_cache_scan_mask(const int64_t* mask, int64_t mask_stride, int32_t* pos, int32_t* count, int B, int64_t N,
                        moa_stream_t stream) {
  using namespace moa;
  MOA_REQUIRE(mask && pos && count, "cache_scan_mask: null pointer");
  MOA_REQUIRE(B > 0 && N > 0 && N < 2147483647LL, "cache_scan_mask: bad shape");
  cache_scan_mask_kernel<<<B, kScanThreads, 0, (cudaStream_t)stream>>>(mask, mask_stride, pos, count, N);
  MOA_CUDA_CHECK(cudaGetLastError());
  return MOA_OK;
}

int moa_cache_fill(const void* k, const void* v, int64_t sb, int64_t sh, int64_t sn, void* k_cache, void* v_cache,
                   const int32_t* pos, const int32_t* count, const int64_t* head_start, int64_t* valid_len,
                   int64_t* update_index, int64_t* mask_cache, const int64_t* static_size, int64_t kv_len, int B,
                   int H, int64_t N, int D, int64_t S, int64_t max_cap, int dtype, moa_stream_t stream) {
  using namespace moa;
  MOA_REQUIRE(k && v && k_cache && v_cache && head_start && valid_len && update_index && static_size,
              "cache_fill: null pointer");
  MOA_REQUIRE((pos == nullptr) == (count == nullptr), "cache_fill: pos and count go together");
  MOA_REQUIRE(B > 0 && H > 0 && N > 0 && S > 0 && max_cap > 0 && B <= 65535 && H <= 65535, "cache_fill: bad shape");
  MOA_REQUIRE(sb % 8 == 0 && sh % 8 == 0 && sn % 8 == 0, "cache_fill: strides must be multiples of 8 elements");
  MOA_REQUIRE(dtype == MOA_F16 || dtype == MOA_BF16, "cache_fill: bad dtype");
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((unsigned)ceil_div64(max_cap + 1, kFillRows), (unsigned)H, (unsigned)B);
  auto kp = (const uint16_t*)k; auto vp = (const uint16_t*)v;
  auto kc = (uint16_t*)k_cache; auto vc = (uint16_t*)v_cache;
  if (D == 128) {
    cache_fill_kernel<128><<<grid, kFillThreads, 0, st>>>(kp, vp, sb, sh, sn, kc, vc, pos, count, head_start,
                                                          update_index, mask_cache, static_size, kv_len, H, N, S);
  } else if (D == 64) {
    cache_fill_kernel<64><<<grid, kFillThreads, 0, st>>>(kp, vp, sb, sh, sn, kc, vc, pos, count, head_start,
                                                         update_index, mask_cache, static_size, kv_len, H, N, S);
  } else {
    set_error_text("cache_fill: head_dim must be 64 or 128");
    return MOA_ERR_UNSUPPORTED;
  }
  MOA_CUDA_CHECK(cudaGetLastError());
  const int64_t nbh = (int64_t)B * H;
  cache_fill_finalize_kernel<<<(unsigned)ceil_div64(nbh, 128), 128, 0, st>>>(count, head_start, valid_len,
                                                                             update_index, static_size, kv_len, B, H,
                                                                             N, S);
  MOA_CUDA_CHECK(cudaGetLastError());
  return MOA_OK;
}

}  // extern "C"
