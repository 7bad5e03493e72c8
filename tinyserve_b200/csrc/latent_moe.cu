// Kernels around latent attention, around a mixture of experts, and the norm of a block that
// norms its sub-layers' outputs as well as their inputs.  Everything here is 32-bit arithmetic
// on rows; inputs and outputs are float or bfloat16.
//
//  * ts_normed_add_rmsnorm: residual += y / rms(y) * w_post; out = residual / rms(residual) * w_pre
//    (the second norm of one sub-layer and the first of the next in one pass over the row).
//  * ts_latent_prepare: from one fused projection of a token, the query latent (RMS-normed) and
//    what the cache keeps of the token: the RMS-normed key/value latent followed by the one
//    rotated key part that all heads share, written to the token's cache slot.
//  * ts_latent_query: the query rows the attention kernel reads: per head the query carried into
//    the latent space followed by its rotated part, padded with zeros to the stored width.
//  * ts_gate_heads: out[t, h, :] = x[h, t, :] * sigmoid(gate[t, h, :]).
//  * ts_moe_route: softmax over all experts of a token's router logits; the `top` largest keep
//    their probability (as it is, or with `renorm` divided by the sum of the kept ones, which is the
//    softmax over the chosen logits alone), the others get zero.
//  * ts_moe_activate: a[t, e, :] <- act(a[t, e, :]) * gate[t, e], act = relu squared.
//  * ts_moe_route_scored: scores s = sigmoid(z); the choice is made on s + correction, among the
//    experts of the `keep` best of `groups` equal groups of neighbours (a group's score: the sum of
//    its two largest choice scores); the `top` chosen experts keep s as their weight.
//  * ts_moe_gated_activate: out[t, e, :] = gated_value(a[t, e, :ff], a[t, e, ff:]) * gate[t, e].
//  * ts_moe_group, ts_moe_gather, ts_moe_combine: the tokens of a step sorted by expert (every
//    expert's rows a run that starts at a multiple of 16), their inputs gathered into that order,
//    and the experts' outputs added back per token with the router's weights in 32-bit.
//  * ts_batched_matmul: C[b] = A[b] B[b] with 32-bit FMA (any strides), chains of 64 k.
#include "common.cuh"

TS_DEFINE_LAST_ERROR()

namespace {

// ------------------------------------------------------------------ post-norm, add, pre-norm
template <typename T>
__global__ void normed_add_rmsnorm_kernel(const T* __restrict__ y, VecParam w_post, float* __restrict__ residual,
                                          VecParam w_pre, float eps_post, float eps_pre, T* __restrict__ out,
                                          const int* __restrict__ rows, int n, int write_residual) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const size_t m = rows ? rows[blockIdx.x] : blockIdx.x;
  float* r = residual + m * n;
  float sq = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float v = to_f32<T>(y[m * n + c]);
    row[c] = v;
    sq += v * v;
  }
  const float rstd_y = rsqrtf(block_sum(sq, scratch) / (float)n + eps_post);
  sq = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float v = r[c] + row[c] * rstd_y * w_post[c];
    if (write_residual) r[c] = v;
    row[c] = v;
    sq += v * v;
  }
  if (out == nullptr) return;
  const float rstd = rsqrtf(block_sum(sq, scratch) / (float)n + eps_pre);
  T* o = out + (size_t)blockIdx.x * n;
  for (int c = threadIdx.x; c < n; c += blockDim.x) o[c] = from_f32<T>(row[c] * rstd * w_pre[c]);
}

// ------------------------------------------------------------------ latent attention: what a token leaves
struct LatentPrepare {
  const void* proj; long long ld;         // [T, >= q_rank + kv_rank + rot_dim]: query latent | kv latent | shared key part
  int q_rank, kv_rank, rot_dim, stored;   // stored: width of a cache row, >= kv_rank + rot_dim
  int has_kv;                             // 0: the projection holds the query latent only
  int interleaved;                        // pairs (2j, 2j + 1) instead of (j, j + rot_dim / 2)
  VecParam q_weight, kv_weight;
  float eps;
  const int* positions; const float* cos; const float* sin;   // tables [positions, rot_dim / 2]
  void* q_latent;                         // [T, q_rank]
  void* cache; const int* slot_mapping;   // [slots, stored]; slot < 0: nothing is written
};

template <typename T>
__global__ void latent_prepare_kernel(LatentPrepare p) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  const T* x = static_cast<const T*>(p.proj) + t * p.ld;
  float sq = 0.f;
  for (int c = threadIdx.x; c < p.q_rank; c += blockDim.x) {
    const float v = to_f32<T>(x[c]);
    sq += v * v;
  }
  const float rq = rsqrtf(block_sum(sq, scratch) / (float)p.q_rank + p.eps);
  T* ql = static_cast<T*>(p.q_latent) + t * p.q_rank;
  for (int c = threadIdx.x; c < p.q_rank; c += blockDim.x) ql[c] = from_f32<T>(to_f32<T>(x[c]) * rq * p.q_weight[c]);
  if (!p.has_kv) return;
  const int slot = p.slot_mapping ? p.slot_mapping[t] : -1;
  if (slot < 0) return;
  const T* kv = x + p.q_rank;
  sq = 0.f;
  for (int c = threadIdx.x; c < p.kv_rank; c += blockDim.x) {
    const float v = to_f32<T>(kv[c]);
    sq += v * v;
  }
  const float rk = rsqrtf(block_sum(sq, scratch) / (float)p.kv_rank + p.eps);
  T* dst = static_cast<T*>(p.cache) + (size_t)slot * p.stored;
  for (int c = threadIdx.x; c < p.kv_rank; c += blockDim.x) dst[c] = from_f32<T>(to_f32<T>(kv[c]) * rk * p.kv_weight[c]);
  const int half = p.rot_dim >> 1;
  const size_t at = (size_t)p.positions[t] * half;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    const int ia = p.kv_rank + (p.interleaved ? 2 * j : j), ib = p.kv_rank + (p.interleaved ? 2 * j + 1 : j + half);
    const float a = to_f32<T>(kv[ia]), b = to_f32<T>(kv[ib]);
    const float cs = p.cos[at + j], sn = p.sin[at + j];
    dst[ia] = from_f32<T>(a * cs - b * sn);
    dst[ib] = from_f32<T>(b * cs + a * sn);
  }
  for (int c = p.kv_rank + p.rot_dim + threadIdx.x; c < p.stored; c += blockDim.x) dst[c] = from_f32<T>(0.f);
}

// ------------------------------------------------------------------ latent attention: query rows
// out[t, h, :] = [ carried[h, t, :kv_rank] | rotate(q[t, h, dim : dim + rot_dim]) | 0 ]; the rotation pairs
// element j with j + rot_dim / 2, or with `interleaved` element 2j with 2j + 1
template <typename T>
__global__ void latent_query_kernel(const T* __restrict__ carried, const T* __restrict__ q, long long ldq, int H, int dim,
                                    int rot_dim, int kv_rank, int stored, const int* __restrict__ positions,
                                    const float* __restrict__ cos, const float* __restrict__ sin, T* __restrict__ out,
                                    int num_tokens, int interleaved) {
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  const int half = rot_dim >> 1;
  const size_t at = (size_t)positions[t] * half;
  for (int h = blockIdx.y; h < H; h += gridDim.y) {
    const T* src = carried + ((size_t)h * num_tokens + t) * kv_rank;
    T* dst = out + (t * H + h) * stored;
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) dst[c] = src[c];
    const T* qr = q + t * ldq + (size_t)h * (dim + rot_dim) + dim;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;
      const float a = to_f32<T>(qr[ia]), b = to_f32<T>(qr[ib]);
      const float cs = cos[at + j], sn = sin[at + j];
      dst[kv_rank + ia] = from_f32<T>(a * cs - b * sn);
      dst[kv_rank + ib] = from_f32<T>(b * cs + a * sn);
    }
    for (int c = kv_rank + rot_dim + threadIdx.x; c < stored; c += blockDim.x) dst[c] = from_f32<T>(0.f);
  }
}

// out[t, h * n + c] = x[h, t, c] * sigmoid(gate[t * ldg + h * n + c]) (gate null: the heads are only laid side by side)
template <typename T>
__global__ void gate_heads_kernel(const T* __restrict__ x, const T* __restrict__ gate, long long ldg, T* __restrict__ out,
                                  int H, int n, int num_tokens) {
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < H * n; i += blockDim.x) {
    const int h = i / n, c = i % n;
    const T v = x[((size_t)h * num_tokens + t) * n + c];
    out[t * H * n + i] = gate ? from_f32<T>(to_f32<T>(v) / (1.f + expf(-to_f32<T>(gate[t * ldg + i])))) : v;
  }
}

// ------------------------------------------------------------------ mixture of experts
// a warp per token: probabilities of all experts, the `top` largest kept (ties: the lower number)
// one warp, one token: z [E] logits -> g [E] (global or shared memory)
// `bias` [E] (or null) is added to the logits first, in 32-bit
__device__ __forceinline__ void route_token(const float* __restrict__ z, float* g, int E, int top, int lane,
                                            int renorm = 0, const float* __restrict__ bias = nullptr) {
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e] + (bias ? bias[e] : 0.f));
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) sum += expf(z[e] + (bias ? bias[e] : 0.f) - mx);
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  for (int e = lane; e < E; e += 32) g[e] = -expf(z[e] + (bias ? bias[e] : 0.f) - mx) * inv;      // negative: not chosen yet
  __syncwarp();
  for (int k = 0; k < top; ++k) {
    float best = 0.f;                 // the largest probability among those not chosen yet
    int best_e = E;
    for (int e = lane; e < E; e += 32) {
      const float v = -g[e];
      if (v > best || (v == best && v > 0.f && e < best_e)) { best = v; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if (lane == 0 && best_e < E) g[best_e] = best;
    __syncwarp();
  }
  for (int e = lane; e < E; e += 32)
    if (g[e] < 0.f) g[e] = 0.f;
  if (renorm) {      // the softmax over the chosen logits alone: their probabilities over their own sum
    __syncwarp();
    float chosen = 0.f;
    for (int e = lane; e < E; e += 32) chosen += g[e];
    chosen = warp_sum(chosen);
    const float r = 1.f / chosen;
    for (int e = lane; e < E; e += 32) g[e] *= r;
  }
}

// One warp, one token.  z [E] logits, corr [E] or null -> g [E]: sigmoid(z) for the chosen experts,
// zero for the others.  scratch: 2 E + 2 groups floats of this warp's own.  Ties go to the lower number.
__device__ __forceinline__ void warp_argmax(float& best, int& at) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oa = __shfl_xor_sync(0xffffffffu, at, o);
    if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
  }
}
__device__ __forceinline__ void route_token_scored(const float* __restrict__ z, const float* __restrict__ corr, float* g,
                                                   float* scratch, int E, int top, int groups, int keep, int lane) {
  float* choice = scratch;            // [E] choice scores; minus infinity once taken or shut out
  float* taken = scratch + E;         // [E] 1 for a chosen expert
  float* gscore = taken + E;          // [groups]
  float* gopen = gscore + groups;     // [groups] 1 for a group whose experts may be chosen
  for (int e = lane; e < E; e += 32) {
    const float s = 1.f / (1.f + expf(-z[e]));
    g[e] = s;
    choice[e] = s + (corr ? corr[e] : 0.f);
    taken[e] = 0.f;
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int per = E / groups;
    for (int grp = 0; grp < groups; ++grp) {
      float b1 = -INFINITY; int a1 = E;
      for (int e = lane; e < per; e += 32) {
        const float v = choice[grp * per + e];
        if (v > b1) { b1 = v; a1 = e; }
      }
      warp_argmax(b1, a1);
      float b2 = -INFINITY; int a2 = E;
      for (int e = lane; e < per; e += 32) {
        const float v = choice[grp * per + e];
        if (e != a1 && v > b2) { b2 = v; a2 = e; }
      }
      warp_argmax(b2, a2);
      if (lane == 0) {
        gscore[grp] = per > 1 ? b1 + b2 : b1;
        gopen[grp] = 0.f;
      }
    }
    __syncwarp();
    for (int k = 0; k < keep; ++k) {
      float best = -INFINITY; int at = groups;
      for (int grp = lane; grp < groups; grp += 32)
        if (gopen[grp] == 0.f && (gscore[grp] > best || at == groups)) { best = gscore[grp]; at = grp; }
      // (a group of score minus infinity is still a group: `at` starts at the first open one)
      warp_argmax(best, at);
      if (lane == 0 && at < groups) gopen[at] = 1.f;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gopen[e / per] == 0.f) choice[e] = -INFINITY;
    __syncwarp();
  }
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY; int at = E;
    for (int e = lane; e < E; e += 32)
      if (choice[e] > best) { best = choice[e]; at = e; }
    warp_argmax(best, at);
    if (lane == 0 && at < E) { taken[at] = 1.f; choice[at] = -INFINITY; }
    __syncwarp();
  }
  for (int e = lane; e < E; e += 32)
    if (taken[e] == 0.f) g[e] = 0.f;
}

__global__ void moe_route_scored_kernel(const float* __restrict__ logits, const float* __restrict__ corr,
                                        float* __restrict__ gates, int num_tokens, int E, int top, int groups, int keep) {
  extern __shared__ float route_scratch[];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= num_tokens) return;
  route_token_scored(logits + (size_t)t * E, corr, gates + (size_t)t * E, route_scratch + (size_t)warp * (2 * E + 2 * groups), E,
                     top, groups, keep, lane);
}

// out[r, e * ff + j] = gated_value(a[r, e * 2 ff + j], a[r, e * 2 ff + ff + j]) * gates[r, e] (gates null: 1)
// With `logits` (and top > 0) in place of gates every block routes its row itself first (its first
// warp, into shared memory), as ts_moe_route does: one launch for the router's softmax, its choice
// and the activation.
template <typename T>
__global__ void moe_gated_activate_kernel(const T* __restrict__ a, const float* __restrict__ gates, int E, int ff,
                                          T* __restrict__ out, int act, float limit, const float* __restrict__ logits,
                                          const float* __restrict__ bias, int top, int renorm) {
  extern __shared__ float routed[];      // [E] when the kernel routes
  pdl_trigger();
  pdl_wait();
  const size_t r = blockIdx.x;
  if (logits) {
    if (threadIdx.x < 32) route_token(logits + r * E, routed, E, top, threadIdx.x, renorm, bias);
    __syncthreads();
    gates = routed - r * E;              // the loop below indexes gates[r * E + e]
  }
  const T* row = a + r * (size_t)E * 2 * ff;
  T* dst = out + r * (size_t)E * ff;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < E * ff; i += gridDim.y * blockDim.x) {
    const int e = i / ff, j = i % ff;
    const float g = gates ? gates[r * E + e] : 1.f;
    float y = 0.f;
    if (g != 0.f) {
      const float gate = to_f32<T>(row[(size_t)e * 2 * ff + j]), up = to_f32<T>(row[(size_t)e * 2 * ff + ff + j]);
      y = gated_value(gate, up, act, limit) * g;
    }
    dst[i] = from_f32<T>(y);
  }
}

__global__ void moe_route_kernel(const float* __restrict__ logits, float* __restrict__ gates, int num_tokens, int E, int top,
                                 int renorm, const float* __restrict__ bias) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= num_tokens) return;
  route_token(logits + (size_t)t * E, gates + (size_t)t * E, E, top, lane, renorm, bias);
}

// 16 bytes of a row as floats and back
template <typename T> struct Chunk { static constexpr int N = 16 / sizeof(T); };
template <typename T>
__device__ __forceinline__ void chunk_load(const T* p, float (&v)[Chunk<T>::N]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < Chunk<T>::N; ++i) v[i] = to_f32<T>(e[i]);
}
template <typename T>
__device__ __forceinline__ void chunk_store(T* p, const float (&v)[Chunk<T>::N]) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < Chunk<T>::N; ++i) e[i] = from_f32<T>(v[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// a[t, e * ff + j] <- relu(a)^2 * gates[t, e]; VEC: 16 bytes a thread (ff a multiple of the chunk)
// With `logits` (and top > 0) the block routes its token itself first (its first warp, into shared
// memory): one launch for the router's softmax, its choice and the activation.
template <typename T, bool VEC>
__global__ void moe_activate_kernel(T* __restrict__ a, const float* __restrict__ gates, int E, int ff,
                                    const float* __restrict__ logits, int top) {
  extern __shared__ float routed[];      // [E] when the kernel routes
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  T* row = a + t * (size_t)E * ff;
  if (logits) {
    if (threadIdx.x < 32) route_token(logits + t * E, routed, E, top, threadIdx.x);
    __syncthreads();
    gates = routed - t * E;              // the loops below index gates[t * E + e]
  }
  if constexpr (VEC) {
    constexpr int N = Chunk<T>::N;
    const int per_expert = ff / N;
    for (int c = threadIdx.x; c < E * per_expert; c += blockDim.x) {
      const float g = gates ? gates[t * E + c / per_expert] : 1.f;
      float v[N];
      chunk_load<T>(row + (size_t)c * N, v);
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const float r = fmaxf(v[i], 0.f);
        v[i] = g == 0.f ? 0.f : r * r * g;
      }
      chunk_store<T>(row + (size_t)c * N, v);
    }
  } else {
    for (int i = threadIdx.x; i < E * ff; i += blockDim.x) {
      const float g = gates ? gates[t * E + i / ff] : 1.f;
      const float v = fmaxf(to_f32<T>(row[i]), 0.f);
      row[i] = from_f32<T>(g == 0.f ? 0.f : v * v * g);
    }
  }
}

// Rows by expert.  One block: counts per expert, the runs' starts (each a multiple of ALIGN rows),
// then a row for every (token, expert) pair with a gate above zero.  Within a run the rows are in
// the order the threads arrive; a row's result does not depend on its place.
constexpr int GROUP_ALIGN = 16;
__global__ void __launch_bounds__(1024) moe_group_kernel(const float* __restrict__ gates, int num_tokens, int E,
                                                         int* __restrict__ row_token, int* __restrict__ pair_row,
                                                         int* __restrict__ ends, int capacity) {
  extern __shared__ int sh[];          // [E] counts, then cursors
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) sh[e] = 0;
  for (int i = threadIdx.x; i < capacity; i += blockDim.x) row_token[i] = -1;
  __syncthreads();
  const int pairs = num_tokens * E;
  for (int i = threadIdx.x; i < pairs; i += blockDim.x)
    if (gates[i] > 0.f) atomicAdd(&sh[i % E], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      const int n = sh[e];
      sh[e] = at;                                        // the run's cursor
      at += (n + GROUP_ALIGN - 1) / GROUP_ALIGN * GROUP_ALIGN;
      ends[e] = at;                                      // the run ends where the next one starts (padding rows are zeros)
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    int row = -1;
    if (gates[i] > 0.f) {
      row = atomicAdd(&sh[i % E], 1);
      row_token[row] = i / E;
    }
    pair_row[i] = row;
  }
}

// x_sorted[row] = x[row_token[row]] (zeros where the row is padding)
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ row_token, T* __restrict__ out, int n) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  const int t = row_token[row];
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(t < 0 ? 0 : t) * n);
  uint4* dst = reinterpret_cast<uint4*>(out + row * n);
  const int chunks = n * (int)sizeof(T) / 16;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) dst[c] = t < 0 ? make_uint4(0u, 0u, 0u, 0u) : src[c];
}

// out[t] = sum_e gates[t, e] * y[pair_row[t, e]] over the experts the token chose, in expert order
template <typename T, bool VEC>
__global__ void moe_combine_kernel(const T* __restrict__ y, const float* __restrict__ gates, const int* __restrict__ pair_row,
                                   T* __restrict__ out, int E, int n) {
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  if constexpr (VEC) {
    // the token's experts first (in expert order), then 16 bytes of every chosen row a thread
    constexpr int N = Chunk<T>::N, MOST = 32;
    __shared__ int rows[MOST];
    __shared__ float weights[MOST];
    __shared__ int count;
    if (threadIdx.x == 0) {
      int k = 0;
      for (int e = 0; e < E && k < MOST; ++e) {
        const int row = pair_row[t * E + e];
        if (row >= 0) { rows[k] = row; weights[k] = gates[t * E + e]; ++k; }
      }
      count = k;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < n / N; c += blockDim.x) {
      float acc[N];
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] = 0.f;
      for (int k = 0; k < count; ++k) {
        float v[N];
        chunk_load<T>(y + (size_t)rows[k] * n + (size_t)c * N, v);
#pragma unroll
        for (int i = 0; i < N; ++i) acc[i] = fmaf(weights[k], v[i], acc[i]);
      }
      chunk_store<T>(out + t * n + (size_t)c * N, acc);
    }
  } else {
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
      float acc = 0.f;
      for (int e = 0; e < E; ++e) {
        const int row = pair_row[t * E + e];
        if (row >= 0) acc = fmaf(gates[t * E + e], to_f32<T>(y[(size_t)row * n + c]), acc);
      }
      out[t * n + c] = from_f32<T>(acc);
    }
  }
}

// ------------------------------------------------------------------ batched 32-bit product
// C[b, m, n] = sum_k A[b, m, k] B[b, k, n]; 32 x 32 tiles, a thread makes a 2 x 2 corner, k in
// chains of 64 whose results are added in order (as the package's FMA product does)
constexpr int BT = 32, BKK = 16;
template <typename T>
__global__ void __launch_bounds__(256) batched_matmul_kernel(const T* __restrict__ A, long long sab, long long sam, long long sak,
                                                             const T* __restrict__ B, long long sbb, long long sbk, long long sbn,
                                                             T* __restrict__ C, int M, int N, int K) {
  __shared__ float As[BKK][BT + 1];
  __shared__ float Bs[BKK][BT + 1];
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.z, m0 = blockIdx.y * BT, n0 = blockIdx.x * BT;
  const T* a = A + (size_t)b * sab;
  const T* w = B + (size_t)b * sbb;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, part[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  for (int k0 = 0; k0 < K; k0 += BKK) {
    for (int i = threadIdx.x; i < BT * BKK; i += 256) {
      const int r = i / BKK, k = i % BKK;
      As[k][r] = (m0 + r < M && k0 + k < K) ? to_f32<T>(a[(size_t)(m0 + r) * sam + (size_t)(k0 + k) * sak]) : 0.f;
      const int kk = i / BT, c = i % BT;
      Bs[kk][c] = (n0 + c < N && k0 + kk < K) ? to_f32<T>(w[(size_t)(k0 + kk) * sbk + (size_t)(n0 + c) * sbn]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BKK; ++k) {
      const float a0 = As[k][ty], a1 = As[k][ty + 16], b0 = Bs[k][tx], b1 = Bs[k][tx + 16];
      part[0][0] = fmaf(a0, b0, part[0][0]); part[0][1] = fmaf(a0, b1, part[0][1]);
      part[1][0] = fmaf(a1, b0, part[1][0]); part[1][1] = fmaf(a1, b1, part[1][1]);
    }
    if ((k0 + BKK) % 64 == 0 || k0 + BKK >= K) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) { acc[i][j] += part[i][j]; part[i][j] = 0.f; }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int m = m0 + ty + 16 * i, n = n0 + tx + 16 * j;
      if (m < M && n < N) C[((size_t)b * M + m) * N + n] = from_f32<T>(acc[i][j]);
    }
}

}  // namespace

TS_EXPORT int ts_normed_add_rmsnorm(int dtype, const void* y, const void* w_post, int w_post_is_f32, float* residual,
                                    const void* w_pre, int w_pre_is_f32, float eps_post, float eps_pre, void* out,
                                    const int* rows, int num_out_rows, int n, int write_residual, cudaStream_t stream) {
  TS_REQUIRE(num_out_rows > 0 && n > 0 && y && residual && w_post, "normed_add_rmsnorm: empty input");
  TS_REQUIRE(out == nullptr || w_pre != nullptr, "normed_add_rmsnorm: an output without a weight");
  const size_t smem = (size_t)n * sizeof(float);
  TS_REQUIRE(smem <= 200 * 1024, "normed_add_rmsnorm: rows of %d elements are too long", n);
  const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
  VecParam wa{w_post, w_post_is_f32}, wb{w_pre, w_pre_is_f32};
  if (dtype == TS_F32) {
    if (smem > 48 * 1024 && cudaFuncSetAttribute(normed_add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return ts_fail("normed_add_rmsnorm: shared memory");
    TS_LAUNCH("normed_add_rmsnorm", normed_add_rmsnorm_kernel<float>, num_out_rows, threads, smem, stream, (const float*)y, wa,
              residual, wb, eps_post, eps_pre, (float*)out, rows, n, write_residual);
  } else if (dtype == TS_BF16) {
    if (smem > 48 * 1024 && cudaFuncSetAttribute(normed_add_rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return ts_fail("normed_add_rmsnorm: shared memory");
    TS_LAUNCH("normed_add_rmsnorm", normed_add_rmsnorm_kernel<__nv_bfloat16>, num_out_rows, threads, smem, stream,
              (const __nv_bfloat16*)y, wa, residual, wb, eps_post, eps_pre, (__nv_bfloat16*)out, rows, n, write_residual);
  } else {
    return ts_fail("normed_add_rmsnorm: unknown dtype %d", dtype);
  }
  return 0;
}

TS_EXPORT int ts_latent_prepare(int dtype, const void* proj, long long ld, int q_rank, int kv_rank, int rot_dim, int stored,
                                int has_kv, const void* q_weight, int q_weight_is_f32, const void* kv_weight,
                                int kv_weight_is_f32, float eps, const int* positions, const float* cos, const float* sin,
                                void* q_latent, void* cache, const int* slot_mapping, int num_tokens, int interleaved,
                                cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && q_rank > 0 && proj && q_weight && q_latent, "latent_prepare: empty input");
  TS_REQUIRE(!has_kv || (kv_rank > 0 && rot_dim >= 0 && rot_dim % 2 == 0 && stored >= kv_rank + rot_dim && kv_weight),
             "latent_prepare: a latent of %d with a rotated part of %d does not fit rows of %d", kv_rank, rot_dim, stored);
  TS_REQUIRE(!has_kv || rot_dim == 0 || (positions && cos && sin), "latent_prepare: rotation without tables");
  LatentPrepare p{proj, ld, q_rank, kv_rank, rot_dim, stored, has_kv, interleaved, VecParam{q_weight, q_weight_is_f32},
                  VecParam{kv_weight, kv_weight_is_f32}, eps, positions, cos, sin, q_latent, cache,
                  cache ? slot_mapping : nullptr};
  const int widest = q_rank > kv_rank ? q_rank : kv_rank;
  const int threads = widest >= 1024 ? 256 : 128;
  if (dtype == TS_F32) TS_LAUNCH("latent_prepare", latent_prepare_kernel<float>, num_tokens, threads, 0, stream, p);
  else if (dtype == TS_BF16) TS_LAUNCH("latent_prepare", latent_prepare_kernel<__nv_bfloat16>, num_tokens, threads, 0, stream, p);
  else return ts_fail("latent_prepare: unknown dtype %d", dtype);
  return 0;
}

TS_EXPORT int ts_latent_query(int dtype, const void* carried, const void* q, long long ldq, int H, int dim, int rot_dim,
                              int kv_rank, int stored, const int* positions, const float* cos, const float* sin, void* out,
                              int num_tokens, int interleaved, cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && H > 0 && kv_rank > 0 && stored >= kv_rank + rot_dim && rot_dim % 2 == 0 && carried && q && out,
             "latent_query: sizes do not fit");
  TS_REQUIRE(rot_dim == 0 || (positions && cos && sin), "latent_query: rotation without tables");
  dim3 grid(num_tokens, H < 16 ? H : 16);
  if (dtype == TS_F32)
    TS_LAUNCH("latent_query", latent_query_kernel<float>, grid, 128, 0, stream, (const float*)carried, (const float*)q, ldq, H, dim,
              rot_dim, kv_rank, stored, positions, cos, sin, (float*)out, num_tokens, interleaved);
  else if (dtype == TS_BF16)
    TS_LAUNCH("latent_query", latent_query_kernel<__nv_bfloat16>, grid, 128, 0, stream, (const __nv_bfloat16*)carried,
              (const __nv_bfloat16*)q, ldq, H, dim, rot_dim, kv_rank, stored, positions, cos, sin, (__nv_bfloat16*)out, num_tokens,
              interleaved);
  else return ts_fail("latent_query: unknown dtype %d", dtype);
  return 0;
}

TS_EXPORT int ts_gate_heads(int dtype, const void* x, const void* gate, long long ldg, void* out, int H, int n, int num_tokens,
                            cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && H > 0 && n > 0 && x && out, "gate_heads: empty input");
  const int threads = H * n >= 1024 ? 256 : 128;
  if (dtype == TS_F32)
    TS_LAUNCH("gate_heads", gate_heads_kernel<float>, num_tokens, threads, 0, stream, (const float*)x, (const float*)gate, ldg,
              (float*)out, H, n, num_tokens);
  else if (dtype == TS_BF16)
    TS_LAUNCH("gate_heads", gate_heads_kernel<__nv_bfloat16>, num_tokens, threads, 0, stream, (const __nv_bfloat16*)x,
              (const __nv_bfloat16*)gate, ldg, (__nv_bfloat16*)out, H, n, num_tokens);
  else return ts_fail("gate_heads: unknown dtype %d", dtype);
  return 0;
}

TS_EXPORT int ts_moe_route(const float* logits, float* gates, int num_tokens, int E, int top, int renorm, const float* bias,
                           cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && E > 0 && top > 0 && top <= E && logits && gates, "moe_route: %d of %d experts", top, E);
  TS_LAUNCH("moe_route", moe_route_kernel, (num_tokens + 3) / 4, 128, 0, stream, logits, gates, num_tokens, E, top, renorm, bias);
  return 0;
}

TS_EXPORT int ts_moe_route_scored(const float* logits, const float* correction, float* gates, int num_tokens, int E, int top,
                                  int groups, int keep, cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && E > 0 && top > 0 && top <= E && logits && gates, "moe_route_scored: %d of %d experts", top, E);
  TS_REQUIRE(groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups && top <= keep * (E / groups),
             "moe_route_scored: %d experts in %d groups, %d kept, %d chosen", E, groups, keep, top);
  const int warps = 4;
  const size_t smem = (size_t)warps * (2 * E + 2 * groups) * sizeof(float);
  TS_REQUIRE(smem <= 48 * 1024, "moe_route_scored: %d experts are too many", E);
  TS_LAUNCH("moe_route_scored", moe_route_scored_kernel, (num_tokens + warps - 1) / warps, warps * 32, smem, stream, logits,
            correction, gates, num_tokens, E, top, groups, keep);
  return 0;
}

TS_EXPORT int ts_moe_gated_activate(int dtype, const void* a, const float* gates, int rows, int E, int ff, void* out,
                                    int act, float limit, const float* logits, const float* bias, int top, int renorm,
                                    cudaStream_t stream) {
  TS_REQUIRE(rows > 0 && E > 0 && ff > 0 && a && out, "moe_gated_activate: empty input");
  TS_REQUIRE(!(gates && logits) && (logits == nullptr || (top > 0 && top <= E && E <= 8192)), "moe_gated_activate: gates or logits with top of %d experts", E);
  const size_t smem = logits ? (size_t)E * sizeof(float) : 0;
  TS_REQUIRE(act >= 0 && act < ACT_COUNT && (act != ACT_BOUNDED_SWISH || limit > 0.f), "moe_gated_activate: activation %d", act);
  // a row's columns over several blocks (four elements a thread), so that a step of few rows still fills the SMs
  const long long tiles = ((long long)E * ff + 1023) / 1024;
  const dim3 grid(rows, (unsigned)(tiles < 64 ? tiles : 64));
  if (dtype == TS_F32)
    TS_LAUNCH("moe_gated_activate", moe_gated_activate_kernel<float>, grid, 256, smem, stream, (const float*)a, gates, E, ff, (float*)out, act, limit,
              logits, bias, top, renorm);
  else if (dtype == TS_BF16)
    TS_LAUNCH("moe_gated_activate", moe_gated_activate_kernel<__nv_bfloat16>, grid, 256, smem, stream, (const __nv_bfloat16*)a, gates, E, ff,
              (__nv_bfloat16*)out, act, limit, logits, bias, top, renorm);
  else return ts_fail("moe_gated_activate: unknown dtype %d", dtype);
  return 0;
}

// gates [tokens, E], or logits [tokens, E] with top > 0 (the kernel routes), or neither (the plain activation)
TS_EXPORT int ts_moe_activate(int dtype, void* a, const float* gates, int num_tokens, int E, int ff, const float* logits,
                              int top, cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && E > 0 && ff > 0 && a, "moe_activate: empty input");
  TS_REQUIRE(!(gates && logits) && (logits == nullptr || (top > 0 && top <= E && E <= 8192)), "moe_activate: gates or logits with top of %d experts", E);
  const size_t smem = logits ? (size_t)E * sizeof(float) : 0;
  const bool vec = (uintptr_t)a % 16 == 0 && ff % (dtype == TS_F32 ? 4 : 8) == 0;
  if (dtype == TS_F32) {
    if (vec) TS_LAUNCH("moe_activate", (moe_activate_kernel<float, true>), num_tokens, 256, smem, stream, (float*)a, gates, E, ff, logits, top);
    else TS_LAUNCH("moe_activate", (moe_activate_kernel<float, false>), num_tokens, 256, smem, stream, (float*)a, gates, E, ff, logits, top);
  } else if (dtype == TS_BF16) {
    if (vec) TS_LAUNCH("moe_activate", (moe_activate_kernel<__nv_bfloat16, true>), num_tokens, 256, smem, stream, (__nv_bfloat16*)a, gates, E, ff, logits, top);
    else TS_LAUNCH("moe_activate", (moe_activate_kernel<__nv_bfloat16, false>), num_tokens, 256, smem, stream, (__nv_bfloat16*)a, gates, E, ff, logits, top);
  } else {
    return ts_fail("moe_activate: unknown dtype %d", dtype);
  }
  return 0;
}

TS_EXPORT int ts_moe_group_align() { return GROUP_ALIGN; }

// row_token [capacity] (capacity >= tokens * top + E * (align - 1)), pair_row [tokens, E], ends [E]
TS_EXPORT int ts_moe_group(const float* gates, int num_tokens, int E, int* row_token, int* pair_row, int* ends, int capacity,
                           cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && E > 0 && E <= 4096 && gates && row_token && pair_row && ends && capacity > 0, "moe_group: empty input");
  TS_LAUNCH("moe_group", moe_group_kernel, 1, 1024, (size_t)E * sizeof(int), stream, gates, num_tokens, E, row_token, pair_row, ends,
            capacity);
  return 0;
}

TS_EXPORT int ts_moe_gather(int dtype, const void* x, const int* row_token, void* out, int rows, int n, cudaStream_t stream) {
  TS_REQUIRE(rows > 0 && n > 0 && x && row_token && out, "moe_gather: empty input");
  TS_REQUIRE(((uintptr_t)x | (uintptr_t)out) % 16 == 0, "moe_gather: operands must be 16-byte aligned");
  if (dtype == TS_F32) {
    TS_REQUIRE(n % 4 == 0, "moe_gather: rows of %d floats are no multiple of 16 bytes", n);
    TS_LAUNCH("moe_gather", moe_gather_kernel<float>, rows, 128, 0, stream, (const float*)x, row_token, (float*)out, n);
  } else if (dtype == TS_BF16) {
    TS_REQUIRE(n % 8 == 0, "moe_gather: rows of %d bfloat16 are no multiple of 16 bytes", n);
    TS_LAUNCH("moe_gather", moe_gather_kernel<__nv_bfloat16>, rows, 128, 0, stream, (const __nv_bfloat16*)x, row_token, (__nv_bfloat16*)out, n);
  } else {
    return ts_fail("moe_gather: unknown dtype %d", dtype);
  }
  return 0;
}

TS_EXPORT int ts_moe_combine(int dtype, const void* y, const float* gates, const int* pair_row, void* out, int num_tokens, int E,
                             int n, cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && E > 0 && n > 0 && y && gates && pair_row && out, "moe_combine: empty input");
  const int threads = n >= 2048 ? 256 : 128;
  // (a token of more than 32 experts takes the plain form)
  const bool vec = ((uintptr_t)y | (uintptr_t)out) % 16 == 0 && n % (dtype == TS_F32 ? 4 : 8) == 0 && E <= 32;
  if (dtype == TS_F32) {
    if (vec) TS_LAUNCH("moe_combine", (moe_combine_kernel<float, true>), num_tokens, threads, 0, stream, (const float*)y, gates, pair_row, (float*)out, E, n);
    else TS_LAUNCH("moe_combine", (moe_combine_kernel<float, false>), num_tokens, threads, 0, stream, (const float*)y, gates, pair_row, (float*)out, E, n);
  } else if (dtype == TS_BF16) {
    if (vec) TS_LAUNCH("moe_combine", (moe_combine_kernel<__nv_bfloat16, true>), num_tokens, threads, 0, stream, (const __nv_bfloat16*)y, gates, pair_row, (__nv_bfloat16*)out, E, n);
    else TS_LAUNCH("moe_combine", (moe_combine_kernel<__nv_bfloat16, false>), num_tokens, threads, 0, stream, (const __nv_bfloat16*)y, gates, pair_row, (__nv_bfloat16*)out, E, n);
  } else {
    return ts_fail("moe_combine: unknown dtype %d", dtype);
  }
  return 0;
}

TS_EXPORT int ts_batched_matmul(int dtype, const void* A, long long sab, long long sam, long long sak, const void* B,
                                long long sbb, long long sbk, long long sbn, void* C, int batch, int M, int N, int K,
                                cudaStream_t stream) {
  TS_REQUIRE(batch > 0 && M > 0 && N > 0 && K > 0 && A && B && C, "batched_matmul: empty operand");
  dim3 grid((N + BT - 1) / BT, (M + BT - 1) / BT, batch);
  TS_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "batched_matmul: grid too large");
  if (dtype == TS_F32)
    TS_LAUNCH("batched_matmul", batched_matmul_kernel<float>, grid, 256, 0, stream, (const float*)A, sab, sam, sak, (const float*)B,
              sbb, sbk, sbn, (float*)C, M, N, K);
  else if (dtype == TS_BF16)
    TS_LAUNCH("batched_matmul", batched_matmul_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)A, sab, sam, sak,
              (const __nv_bfloat16*)B, sbb, sbk, sbn, (__nv_bfloat16*)C, M, N, K);
  else return ts_fail("batched_matmul: unknown dtype %d", dtype);
  return 0;
}
