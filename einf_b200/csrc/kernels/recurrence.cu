// Mixers that carry a state of fixed size per request instead of keys and values: a linear
// recurrence over outer products (linear attention with a decay per head; the state-space
// recurrence of Mamba-2 in its recurrent form), the short causal convolution in front of it, and
// the gated norm behind it.  State lives in 32-bit floats in a slot per request
// (state[slot * row_stride + ...]); a request without a slot (-1: padding of a decode graph) reads
// zeros and writes nothing.  The step's tokens are packed request by request, q_start[r] ..
// q_start[r + 1], so a prompt portion and a single decoded token take the same code and the same
// order of additions: what a position computes does not depend on how the prompt was cut.
#include "common.cuh"

namespace einf {

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// ---------------------------------------------------------------------------
// Causal convolution per channel over the tokens of each request, bias, SiLU:
//   out[t, c] = silu(bias[c] + sum_j w[c, j] * in[t - (taps - 1) + j, c]),  j = 0 .. taps-1,
// where inputs before the portion come from the request's convolution state (its last taps-1
// inputs, oldest first, [taps-1, channels] floats; zeros after a fresh start).  The same launch
// turns the raw step sizes of `heads` further columns into
//   dt = softplus(raw + dt_bias[h])   and   decay = exp(-exp(a_log[h]) * dt)
// in 32-bit (columns channels .. channels+heads of the work; `in` holds them at dt_offset).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void conv_silu_kernel(const T* __restrict__ in, long long in_stride, const float* __restrict__ weight,
                                 const float* __restrict__ bias, const float* __restrict__ conv_state,
                                 long long state_stride, const int* __restrict__ seq_of_token,
                                 const int* __restrict__ q_start, const int* __restrict__ state_slots, int num_slots,
                                 T* __restrict__ out, int channels, int taps, int num_tokens,
                                 const T* __restrict__ dt_in, const float* __restrict__ dt_bias,
                                 const float* __restrict__ a_log, float* __restrict__ dt_out,
                                 float* __restrict__ decay_out, int heads) {
  pdl_launch_dependents();
  pdl_wait();
  const int columns = channels + heads;
  const long long total = (long long)num_tokens * columns;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / columns);
    const int c = (int)(idx - (long long)t * columns);
    if (c >= channels) {
      const int h = c - channels;
      const float dt = softplus_f(to_float(dt_in[(long long)t * in_stride + h]) + dt_bias[h]);
      dt_out[(long long)t * heads + h] = dt;
      decay_out[(long long)t * heads + h] = expf(-expf(a_log[h]) * dt);
      continue;
    }
    const int r = seq_of_token[t];
    const int first = q_start[r];
    const int slot = state_slots[r];
    const float* state = (slot >= 0 && slot < num_slots) ? conv_state + (long long)slot * state_stride : nullptr;
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int u = t - (taps - 1) + j;       // packed index of the input, if it is in this step
      float v;
      if (u >= first) v = to_float(in[(long long)u * in_stride + c]);
      else v = state ? state[(long long)(taps - 1 - (first - u)) * channels + c] : 0.f;
      acc = fmaf(weight[(long long)c * taps + j], v, acc);
    }
    out[(long long)t * channels + c] = from_float<T>(silu_f(acc));
  }
}

// After the convolution: the request's last taps-1 inputs become its convolution state (a portion
// shorter than that keeps the tail of the old state in front).  One thread per (request, channel).
constexpr int kMaxTaps = 16;
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ in, long long in_stride, float* __restrict__ conv_state,
                                         long long state_stride, const int* __restrict__ q_start,
                                         const int* __restrict__ state_slots, int num_slots, int channels, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = state_slots[r];
  if (c >= channels || slot < 0 || slot >= num_slots) return;
  const int first = q_start[r], count = q_start[r + 1] - first;
  float* state = conv_state + (long long)slot * state_stride;
  const int keep = taps - 1;
  float fresh[kMaxTaps];
#pragma unroll
  for (int u = 0; u < kMaxTaps; ++u) {
    if (u < keep) {
      const int rel = count - keep + u;      // index among the step's tokens of this request
      fresh[u] = rel >= 0 ? to_float(in[(long long)(first + rel) * in_stride + c]) : state[(long long)(u + count) * channels + c];
    }
  }
#pragma unroll
  for (int u = 0; u < kMaxTaps; ++u)
    if (u < keep) state[(long long)u * channels + c] = fresh[u];
}

// ---------------------------------------------------------------------------
// The recurrence.  Per request and head, with S a [dim, vdim] matrix of floats:
//   S <- a_t S + k_t (s_t v_t)^T,      y_t = S^T q_t + skip_h v_t
// a_t is a constant per head (head_decay) or a value per token and head (token_decay), s_t a
// value per token and head (token_scale) or 1; query and key head of head h is h / (heads /
// groups).  With `act` the inputs pass SiLU as they are read.  q, k, v are rows of some wider
// matrix: element (t, head, i) of q is q[t * q_stride + head * dim + i].
//
// A thread owns kRows consecutive rows of one column of S; the 2^n lanes that share a column
// (lanes_per_column >= dim / kRows) sit kColumns apart in a warp so that loads and stores of S are
// contiguous over the columns, and add their parts of y with shuffles.  Tokens are taken one
// after the other: the order of the additions is the same for a whole prompt, for portions and
// for single tokens.
// ---------------------------------------------------------------------------
constexpr int kRows = 16;
constexpr int kRecurrenceThreads = 128;

struct RecurrenceArgs {
  const void* q; const void* k; const void* v;
  long long q_stride, k_stride, v_stride;
  const float* head_decay; const float* token_decay; const float* token_scale; const float* skip;
  float* state; long long state_stride;
  const int* q_start; const int* state_slots;
  float* y;
  int num_slots, heads, groups, dim, vdim, act, lanes_per_column, vector_loads;
};

template <typename T>
__device__ __forceinline__ void load_rows(const T* __restrict__ p, int r0, int dim, bool vectors, bool act,
                                          float (&out)[kRows]) {
  if (vectors && r0 + kRows <= dim) {
    constexpr int kPerVec = 16 / sizeof(T);
#pragma unroll
    for (int i = 0; i < kRows; i += kPerVec) {
      const uint4 raw = *reinterpret_cast<const uint4*>(p + r0 + i);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int u = 0; u < kPerVec; ++u) out[i + u] = to_float(e[u]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < kRows; ++i) out[i] = (r0 + i < dim) ? to_float(p[r0 + i]) : 0.f;
  }
  if (act) {
#pragma unroll
    for (int i = 0; i < kRows; ++i) out[i] = silu_f(out[i]);
  }
}

template <typename T>
__global__ void __launch_bounds__(kRecurrenceThreads)
linear_recurrence_kernel(const RecurrenceArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int lanes = a.lanes_per_column;          // a power of two, 1 .. 32
  const int columns_per_warp = 32 / lanes;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int part = lane / columns_per_warp;       // which rows of the column
  const int column = (blockIdx.x * (kRecurrenceThreads / 32) + warp) * columns_per_warp + (lane % columns_per_warp);
  const int head = blockIdx.y, r = blockIdx.z;
  const int group = head / (a.heads / a.groups);
  const int first = a.q_start[r], last = a.q_start[r + 1];
  const int slot = a.state_slots[r];
  const bool live = column < a.vdim;
  const int col = live ? column : a.vdim - 1;     // idle lanes follow along and write nothing
  const int r0 = part * kRows;
  const bool vectors = a.vector_loads != 0;
  const bool act = a.act != 0;

  float* state = (slot >= 0 && slot < a.num_slots)
      ? a.state + (long long)slot * a.state_stride + ((long long)head * a.dim) * a.vdim + col : nullptr;
  float S[kRows];
#pragma unroll
  for (int i = 0; i < kRows; ++i) S[i] = (state && r0 + i < a.dim) ? state[(long long)(r0 + i) * a.vdim] : 0.f;

  const T* q = (const T*)a.q + (long long)group * a.dim;
  const T* k = (const T*)a.k + (long long)group * a.dim;
  const T* v = (const T*)a.v + (long long)head * a.vdim + col;
  const float constant_decay = a.head_decay ? a.head_decay[head] : 1.f;
  const float skip = a.skip ? a.skip[head] : 0.f;

  float kn[kRows], qn[kRows], vn = 0.f, an = constant_decay, sn = 1.f;
  if (first < last) {
    load_rows(k + (long long)first * a.k_stride, r0, a.dim, vectors, act, kn);
    load_rows(q + (long long)first * a.q_stride, r0, a.dim, vectors, act, qn);
    vn = to_float(v[(long long)first * a.v_stride]);
    if (act) vn = silu_f(vn);
    if (a.token_decay) an = a.token_decay[(long long)first * a.heads + head];
    if (a.token_scale) sn = a.token_scale[(long long)first * a.heads + head];
  }
  for (int t = first; t < last; ++t) {
    float kc[kRows], qc[kRows];
#pragma unroll
    for (int i = 0; i < kRows; ++i) { kc[i] = kn[i]; qc[i] = qn[i]; }
    const float vc = vn, ac = an, sc = sn;
    if (t + 1 < last) {      // the next token's inputs are on their way while this one is added
      load_rows(k + (long long)(t + 1) * a.k_stride, r0, a.dim, vectors, act, kn);
      load_rows(q + (long long)(t + 1) * a.q_stride, r0, a.dim, vectors, act, qn);
      vn = to_float(v[(long long)(t + 1) * a.v_stride]);
      if (act) vn = silu_f(vn);
      if (a.token_decay) an = a.token_decay[(long long)(t + 1) * a.heads + head];
      if (a.token_scale) sn = a.token_scale[(long long)(t + 1) * a.heads + head];
    }
    const float sv = sc * vc;
    float y = 0.f;
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
      S[i] = fmaf(ac, S[i], kc[i] * sv);
      y = fmaf(S[i], qc[i], y);
    }
    for (int o = columns_per_warp; o < 32; o <<= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
    if (live && part == 0) a.y[((long long)t * a.heads + head) * a.vdim + col] = y + skip * vc;
  }
  if (state && live && first < last) {
#pragma unroll
    for (int i = 0; i < kRows; ++i)
      if (r0 + i < a.dim) state[(long long)(r0 + i) * a.vdim] = S[i];
  }
}

// ---------------------------------------------------------------------------
// Gate and norm behind a recurrence.  y [T, width] floats, gate rows of some wider matrix
// (gate[t * gate_stride + i]), weight [width] floats; the row is cut into `parts` equal parts,
// each divided by its own root mean square (eps inside the root), in 32-bit.
//   gate_first:  u = y * g(gate);  out = u / rms(u) * weight          (gate before the norm)
//   otherwise:   out = y / rms(y) * weight * g(gate)                  (gate after the norm)
// g is SiLU (gate_kind 0) or the logistic sigmoid (1).  One CTA per (token, part).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gated_norm_kernel(const float* __restrict__ y, const T* __restrict__ gate, long long gate_stride,
                                  const float* __restrict__ weight, T* __restrict__ out, int width, int parts,
                                  float eps, int gate_first, int gate_kind) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x / parts, part = blockIdx.x - t * parts;
  const int size = width / parts, base = part * size;
  const float* row = y + (long long)t * width + base;
  const T* g_row = gate + (long long)t * gate_stride + base;
  float ss = 0.f;
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    float u = row[i];
    if (gate_first) {
      const float g = to_float(g_row[i]);
      u *= gate_kind == 0 ? silu_f(g) : 1.f / (1.f + expf(-g));
    }
    ss += u * u;
  }
  const float factor = rsqrtf(block_sum(ss, scratch) / (float)size + eps);
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    const float g = to_float(g_row[i]);
    const float gv = gate_kind == 0 ? silu_f(g) : 1.f / (1.f + expf(-g));
    float u = row[i];
    if (gate_first) u = (u * gv) * factor * weight[base + i];
    else u = u * factor * weight[base + i] * gv;
    out[(long long)t * width + base + i] = from_float<T>(u);
  }
}

}  // namespace einf

using namespace einf;

extern "C" int einf_conv_silu(const void* in, int dtype, long long in_stride, const float* weight, const float* bias,
                              float* conv_state, long long state_stride, const int* seq_of_token, const int* q_start,
                              const int* state_slots, int num_slots, int num_requests, void* out, int channels,
                              int taps, int num_tokens, const void* dt_in, const float* dt_bias, const float* a_log,
                              float* dt_out, float* decay_out, int heads, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (taps < 1 || taps > kMaxTaps || channels <= 0 || num_requests > 65535) return (int)cudaErrorInvalidValue;
  const int threads = 256;
  const long long total = (long long)num_tokens * (channels + heads);
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  EINF_DISPATCH_2(dtype, T, {
    cudaError_t e = launch_pdl(conv_silu_kernel<T>, (int)blocks, threads, 0, stream, (const T*)in, in_stride, weight,
                               bias, (const float*)conv_state, state_stride, seq_of_token, q_start, state_slots,
                               num_slots, (T*)out, channels, taps, num_tokens, (const T*)dt_in, dt_bias, a_log, dt_out,
                               decay_out, heads);
    if (e != cudaSuccess || taps == 1) return (int)e;
    const dim3 grid((channels + 127) / 128, num_requests);
    return (int)launch_pdl(conv_state_update_kernel<T>, grid, 128, 0, stream, (const T*)in, in_stride, conv_state,
                           state_stride, q_start, state_slots, num_slots, channels, taps);
  })
}

extern "C" int einf_linear_recurrence(const void* q, const void* k, const void* v, int dtype, long long q_stride,
                                      long long k_stride, long long v_stride, const float* head_decay,
                                      const float* token_decay, const float* token_scale, const float* skip,
                                      float* state, long long state_stride, int num_slots, const int* q_start,
                                      const int* state_slots, int num_requests, float* y, int heads, int groups,
                                      int dim, int vdim, int act, cudaStream_t stream) {
  if (num_requests == 0) return 0;
  if (heads <= 0 || groups <= 0 || heads % groups || dim <= 0 || vdim <= 0 || dim > 32 * kRows ||
      heads > 65535 || num_requests > 65535)
    return (int)cudaErrorInvalidValue;
  RecurrenceArgs a;
  a.q = q; a.k = k; a.v = v;
  a.q_stride = q_stride; a.k_stride = k_stride; a.v_stride = v_stride;
  a.head_decay = head_decay; a.token_decay = token_decay; a.token_scale = token_scale; a.skip = skip;
  a.state = state; a.state_stride = state_stride;
  a.q_start = q_start; a.state_slots = state_slots;
  a.y = y;
  a.num_slots = num_slots; a.heads = heads; a.groups = groups; a.dim = dim; a.vdim = vdim; a.act = act;
  int lanes = 1;
  while (lanes * kRows < dim) lanes <<= 1;
  a.lanes_per_column = lanes;
  const int element = dtype == kFloat32 ? 4 : 2;
  const int per_vector = 16 / element;
  a.vector_loads = (dim % per_vector == 0 && q_stride % per_vector == 0 && k_stride % per_vector == 0 &&
                    ((uintptr_t)q & 15) == 0 && ((uintptr_t)k & 15) == 0) ? 1 : 0;
  const int columns_per_block = (kRecurrenceThreads / 32) * (32 / lanes);
  const dim3 grid((vdim + columns_per_block - 1) / columns_per_block, heads, num_requests);
  EINF_DISPATCH_2(dtype, T, {
    return (int)launch_pdl(linear_recurrence_kernel<T>, grid, kRecurrenceThreads, 0, stream, a);
  })
}

extern "C" int einf_gated_norm(const float* y, const void* gate, int dtype, long long gate_stride, const float* weight,
                               void* out, int num_tokens, int width, int parts, float eps, int gate_first,
                               int gate_kind, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (parts <= 0 || width % parts) return (int)cudaErrorInvalidValue;
  const int size = width / parts;
  int threads = 32;
  while (threads < size && threads < 256) threads <<= 1;
  const long long blocks = (long long)num_tokens * parts;
  if (blocks >= (1ll << 31)) return (int)cudaErrorInvalidValue;
  EINF_DISPATCH_2(dtype, T, {
    return (int)launch_pdl(gated_norm_kernel<T>, (int)blocks, threads, 0, stream, y, (const T*)gate, gate_stride, weight,
                           (T*)out, width, parts, eps, gate_first, gate_kind);
  })
}
