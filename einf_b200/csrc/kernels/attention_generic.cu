// Paged causal attention for any batch: prompt portions and single decoded
// tokens alike, float or bfloat16, any head size up to 256 (16-byte loads where
// the size allows them), any number of heads and groups, with an optional
// sliding window, chunked mask and soft cap on the scores.
//
// This is the 32-bit path's attention and the fallback of the bfloat16 path for
// sizes its tensor-core kernels do not cover.  One warp owns one (token, query
// head) row and walks the keys of its request 32 at a time straight from the
// pages named by the block table:
//   scores: lane j computes q . K[j] in 32-bit (q is pre-multiplied by scale)
//   online softmax in 32-bit across the warp (max, exp, sum)
//   output: lane d accumulates sum_j p_j V[j][d] in 32-bit
// (reference for the maths: src/einf/executors/torch/ops/csrc/paged_attention_cuda.cu:74-147
// and flash_attention_cuda.cu:126-195; lower-right causal mask model_runner.py:145.)
// A token at position p of request r sees keys lo..p of r, lo = max(0, p - window + 1); with a
// chunk size c (chunked attention) lo is also at least floor(p / c) * c, the first position of p's
// own chunk, counted from position 0 of the sequence.  With a soft cap z the scaled score s becomes
// z * tanh(s / z) before the softmax.  Keys and values may have different sizes per head.
// With `keep_first` n > 0 a windowed token also sees the first n positions of its sequence
// (j < n), at their true positions.  `value_stride` is the distance between two value rows in
// elements: value_size for a cache of its own, the key size when the values are the leading
// elements of the key rows (a latent cache that holds one row per token for both).
// The kernel exists twice: for sizes up to 256 and for sizes up to 640 (more registers a lane).
#include "common.cuh"

namespace einf {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxHeadSize = 640;

template <typename T>
struct Vec;  // 16-byte vector of T
template <>
struct Vec<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ float get(int i) const { return (&raw.x)[i]; }
};
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ float get(int i) const {
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(&raw);
    return __bfloat162float(p[i]);
  }
};

template <typename T, int kHeadLimit>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_cache,
                               const T* __restrict__ v_cache, const int* __restrict__ block_table,
                               const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                               T* __restrict__ out, int num_rows, int num_heads, int num_kv_heads,
                               int head_size, int value_size, int value_stride, int page_size, int num_pages,
                               int table_width, float scale, int window, int keep_first, int chunk, float softcap,
                               int* status) {
  __shared__ float q_smem[kWarpsPerBlock][kHeadLimit];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerBlock + warp;
  if (row >= num_rows) return;
  const int t = row / num_heads;
  const int h = row - t * num_heads;
  const int kv_head = h / (num_heads / num_kv_heads);
  const int r = seq_of_token[t];
  const int pos = positions[t];
  int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
  const bool vectors = head_size % Vec<T>::N == 0;
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  const int* table = block_table + (size_t)r * table_width;

  const T* q_row = q + (size_t)row * head_size;
  for (int d = lane; d < head_size; d += 32) q_smem[warp][d] = to_float(q_row[d]) * scale;
  __syncwarp();
  const float* qs = q_smem[warp];

  constexpr int kDimsPerLane = kHeadLimit / 32;
  float acc[kDimsPerLane];
#pragma unroll
  for (int i = 0; i < kDimsPerLane; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  bool bad_page = false;

  // Two ranges of keys: the kept first positions below the window (empty without them), then
  // the window itself.
  const int kept = (window > 0 && keep_first > 0) ? min(keep_first, lo) : 0;
  for (int range = kept > 0 ? 0 : 1; range < 2; ++range) {
  const int first = range == 0 ? 0 : lo;
  const int last = range == 0 ? kept - 1 : pos;
  for (int base = first; base <= last; base += 32) {
    const int j = base + lane;
    float s = -INFINITY;
    long long key_row = -1;  // index of the (page, kv_head, slot) row in the caches, or -1
    if (j <= last) {
      const int logical = j / page_size;
      const int page = table[logical];
      if (page < 0 || page >= num_pages) {
        bad_page = true;
      } else {
        key_row = ((long long)page * num_kv_heads + kv_head) * page_size + (j - logical * page_size);
        const T* k_row = k_cache + key_row * head_size;
        float dot = 0.f;
        if (vectors) {
          for (int d = 0; d < head_size; d += Vec<T>::N) {
            Vec<T> kv;
            kv.raw = *reinterpret_cast<const decltype(kv.raw)*>(k_row + d);
#pragma unroll
            for (int e = 0; e < Vec<T>::N; ++e) dot = fmaf(qs[d + e], kv.get(e), dot);
          }
        } else {
          for (int d = 0; d < head_size; ++d) dot = fmaf(qs[d], to_float(k_row[d]), dot);
        }
        s = softcap > 0.f ? softcap * tanhf(dot * inv_cap) : dot;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    // m_new is finite unless every key so far had a bad page (the kept range comes first, so
    // key `pos` itself may still be ahead): then nothing is added.
    const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
    const float correction = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * correction + warp_sum(p);
#pragma unroll
    for (int i = 0; i < kDimsPerLane; ++i) acc[i] *= correction;
    m = m_new;
    const int count = min(32, last - base + 1);
    for (int kk = 0; kk < count; ++kk) {
      const float pj = __shfl_sync(0xffffffffu, p, kk);
      const long long off = __shfl_sync(0xffffffffu, key_row, kk);
      if (off < 0) continue;
      const T* v_row = v_cache + off * value_stride;
#pragma unroll
      for (int i = 0; i < kDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < value_size) acc[i] = fmaf(pj, to_float(v_row[d]), acc[i]);
      }
    }
  }
  }
  if (__any_sync(0xffffffffu, bad_page) && lane == 0) atomicOr(status, kStatusBadPage);
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T* o_row = out + (size_t)row * value_size;
#pragma unroll
  for (int i = 0; i < kDimsPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < value_size) o_row[d] = from_float<T>(acc[i] * inv);
  }
}

}  // namespace einf

using namespace einf;

extern "C" int einf_paged_attention_generic(const void* q, const void* k_cache, const void* v_cache,
                                            int dtype, const int* block_table, const int* seq_of_token,
                                            const int* positions, void* out, int num_tokens,
                                            int num_heads, int num_kv_heads, int head_size, int value_size,
                                            int value_stride, int page_size, int num_pages, int table_width,
                                            float scale, int window, int keep_first, int chunk, float softcap,
                                            int* status, cudaStream_t stream) {
  const int rows = num_tokens * num_heads;
  if (rows == 0) return 0;
  if (head_size > kMaxHeadSize || value_size > kMaxHeadSize || head_size <= 0 || value_size <= 0)
    return (int)cudaErrorInvalidValue;
  const int blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (value_stride < value_size) return (int)cudaErrorInvalidValue;
  EINF_DISPATCH_2(dtype, T, {
    if (head_size <= 256 && value_size <= 256) {
      paged_attention_generic_kernel<T, 256><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(
          (const T*)q, (const T*)k_cache, (const T*)v_cache, block_table, seq_of_token, positions, (T*)out,
          rows, num_heads, num_kv_heads, head_size, value_size, value_stride, page_size, num_pages, table_width,
          scale, window, keep_first, chunk, softcap, status);
    } else {
      paged_attention_generic_kernel<T, kMaxHeadSize><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(
          (const T*)q, (const T*)k_cache, (const T*)v_cache, block_table, seq_of_token, positions, (T*)out,
          rows, num_heads, num_kv_heads, head_size, value_size, value_stride, page_size, num_pages, table_width,
          scale, window, keep_first, chunk, softcap, status);
    }
  })
  return (int)cudaGetLastError();
}
