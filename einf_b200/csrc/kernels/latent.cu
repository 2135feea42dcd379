// Pointwise steps of latent attention: keys and values of a token are one normed latent vector
// c [kv_rank] plus one rotated key part r [rot_dim] shared by all heads; the page cache holds the
// row [c | r] once per token (one key/value "head" of size kv_rank + rot_dim whose first kv_rank
// elements are also the value).  Queries come through a normed latent of their own.
//
//   einf_latent_down_store   from the product [q latent | kv latent | key part] of a token:
//                            RMS norm (weight, eps inside the root) of the query latent -> q_latent_out,
//                            RMS norm of the kv latent and rotation of the key part -> cache row
//   einf_latent_q_store      from the up-projected queries [H, dim + rot_dim]: the unrotated part
//                            -> q_plain [T, H, dim] (it still has to pass the key up-projection),
//                            the rotated part -> q_full [T, H, kv_rank + rot_dim] behind the place
//                            of the absorbed part
//
// Rotation of a pair (u, v) at position p: (u cos a - v sin a, v cos a + u sin a), a = p * inv_freq[i];
// pair i is (i, i + rot_dim / 2), or (2i, 2i + 1) with `interleaved`.  Norms, angles and sums are
// 32-bit; values are rounded once, into the output type.  Inputs may be float32 split-K partial sums.
#include "common.cuh"

namespace einf {

// Sum of the partial sums of one element, added in order; the loads go out eight at a time (a consumer
// of a product that was cut sixteen ways would otherwise pay sixteen round trips one after the other).
template <typename TIn>
__device__ __forceinline__ float sum_parts(const TIn* __restrict__ p, int splits, size_t split_stride) {
  float v = 0.f;
  int s = 0;
  for (; s + 8 <= splits; s += 8) {
    float t[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) t[u] = to_float(p[(size_t)(s + u) * split_stride]);
#pragma unroll
    for (int u = 0; u < 8; ++u) v += t[u];
  }
  if (s < splits) {
    float t[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) t[u] = s + u < splits ? to_float(p[(size_t)(s + u) * split_stride]) : 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) v += t[u];
  }
  return v;
}

__device__ __forceinline__ void pair_of(int i, int half, int interleaved, int* first, int* second) {
  if (interleaved) {
    *first = 2 * i;
    *second = 2 * i + 1;
  } else {
    *first = i;
    *second = i + half;
  }
}

template <typename TIn, typename T>
__global__ void __launch_bounds__(256)
latent_down_store_kernel(const TIn* __restrict__ down, int splits, size_t split_stride, int q_rank, int kv_rank,
                         int rot_dim, const float* __restrict__ q_norm_weight,
                         const float* __restrict__ kv_norm_weight, float eps, const int* __restrict__ positions,
                         const float* __restrict__ inv_freq, int interleaved, const int* __restrict__ slots,
                         T* __restrict__ q_latent_out, T* __restrict__ cache, int page_size, int num_pages,
                         int* status) {
  extern __shared__ float row[];   // [q_rank + kv_rank + rot_dim]
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int width = q_rank + kv_rank + rot_dim;
  const TIn* src = down + (size_t)t * width;
  float ss_q = 0.f, ss_kv = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = sum_parts(src + i, splits, split_stride);
    row[i] = v;
    if (i < q_rank) ss_q += v * v;
    else if (i < q_rank + kv_rank) ss_kv += v * v;
  }
  if (q_rank > 0) {
    const float factor = rsqrtf(block_sum(ss_q, scratch) / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
      q_latent_out[(size_t)t * q_rank + i] = from_float<T>(row[i] * factor * q_norm_weight[i]);
  }
  const float factor = rsqrtf(block_sum(ss_kv, scratch) / (float)kv_rank + eps);   // has barriers: row[] is complete
  const int slot = slots ? slots[t] : -1;
  if (slot < 0) return;
  const int page = slot / page_size, offset = slot - page * page_size;
  if (page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, kStatusBadPage);
    return;
  }
  T* dst = cache + ((size_t)page * page_size + offset) * (kv_rank + rot_dim);
  const float* latent = row + q_rank;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x)
    dst[i] = from_float<T>(latent[i] * factor * kv_norm_weight[i]);
  const float* part = latent + kv_rank;
  const int half = rot_dim >> 1;
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    int a, b;
    pair_of(i, half, interleaved, &a, &b);
    float sn, cs;
    sincosf(pos * inv_freq[i], &sn, &cs);
    const float u = part[a], v = part[b];
    dst[kv_rank + a] = from_float<T>(u * cs - v * sn);
    dst[kv_rank + b] = from_float<T>(v * cs + u * sn);
  }
}

template <typename TIn, typename T>
__global__ void latent_q_store_kernel(const TIn* __restrict__ q, int splits, size_t split_stride, int num_tokens,
                                      int num_heads, int dim, int rot_dim, int kv_rank,
                                      const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                      int interleaved, T* __restrict__ q_plain, T* __restrict__ q_full) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (warp >= (long long)num_tokens * num_heads) return;
  const int t = (int)(warp / num_heads);
  const TIn* src = q + (size_t)warp * (dim + rot_dim);
  T* plain = q_plain + (size_t)warp * dim;
  for (int d = lane; d < dim; d += 32) plain[d] = from_float<T>(sum_parts(src + d, splits, split_stride));
  T* dst = q_full + (size_t)warp * (kv_rank + rot_dim) + kv_rank;
  const int half = rot_dim >> 1;
  const float pos = (float)positions[t];
  for (int i = lane; i < half; i += 32) {
    int a, b;
    pair_of(i, half, interleaved, &a, &b);
    const float u = sum_parts(src + dim + a, splits, split_stride);
    const float v = sum_parts(src + dim + b, splits, split_stride);
    float sn, cs;
    sincosf(pos * inv_freq[i], &sn, &cs);
    dst[a] = from_float<T>(u * cs - v * sn);
    dst[b] = from_float<T>(v * cs + u * sn);
  }
}

}  // namespace einf

using namespace einf;

// down: [T, q_rank + kv_rank + rot_dim] (or `splits` float32 partial sums of it); cache:
// [pages, 1, page_size, kv_rank + rot_dim]; q_latent_out: [T, q_rank] (q_rank may be 0).
extern "C" int einf_latent_down_store(const void* down, int in_dtype, int splits, long long split_stride, int dtype,
                                      int num_tokens, int q_rank, int kv_rank, int rot_dim,
                                      const float* q_norm_weight, const float* kv_norm_weight, float eps,
                                      const int* positions, const float* inv_freq, int interleaved,
                                      const int* slots, void* q_latent_out, void* cache, int page_size,
                                      int num_pages, int* status, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (kv_rank <= 0 || rot_dim < 0 || (rot_dim & 1) || q_rank < 0) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)(q_rank + kv_rank + rot_dim) * sizeof(float);
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  EINF_DISPATCH_2(in_dtype, TIn, {
    EINF_DISPATCH_2(dtype, T, {
      return (int)launch_pdl(latent_down_store_kernel<TIn, T>, num_tokens, 256, smem, stream, (const TIn*)down, splits,
                             (size_t)split_stride, q_rank, kv_rank, rot_dim, q_norm_weight, kv_norm_weight, eps,
                             positions, inv_freq, interleaved, slots, (T*)q_latent_out, (T*)cache, page_size,
                             num_pages, status);
    })
  })
}

// q: [T, H * (dim + rot_dim)] (or partial sums); q_plain: [T, H, dim]; q_full: [T, H, kv_rank + rot_dim],
// of which this writes the last rot_dim elements of every head.
extern "C" int einf_latent_q_store(const void* q, int in_dtype, int splits, long long split_stride, int dtype,
                                   int num_tokens, int num_heads, int dim, int rot_dim, int kv_rank,
                                   const int* positions, const float* inv_freq, int interleaved, void* q_plain,
                                   void* q_full, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const long long warps = (long long)num_tokens * num_heads;
  const int threads = 128;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  if (blocks >= (1ll << 31) || (rot_dim & 1)) return (int)cudaErrorInvalidValue;
  EINF_DISPATCH_2(in_dtype, TIn, {
    EINF_DISPATCH_2(dtype, T, {
      return (int)launch_pdl(latent_q_store_kernel<TIn, T>, (int)blocks, threads, 0, stream, (const TIn*)q, splits,
                             (size_t)split_stride, num_tokens, num_heads, dim, rot_dim, kv_rank, positions, inv_freq,
                             interleaved, (T*)q_plain, (T*)q_full);
    })
  })
}
