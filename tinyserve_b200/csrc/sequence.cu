// Kernels on rows of a step that depend on a token's neighbours in its own sequence, and the
// small 32-bit steps around recurrent mixers.  All arithmetic is 32-bit; inputs and outputs are
// float or bfloat16 (an `is_f32` flag per operand, so that the 32-bit residual stream and the
// projections of the compute type go through the same kernels).
//
//  * ts_add_position_rows: residual[t] += table[positions[t]] (learned positions).
//  * ts_causal_conv: y_t = (x_t +) (bias +) sum_j w[:, j] x_(t - taps + 1 + j) per channel, zeros
//    before a sequence's start, optionally through silu.  The last taps - 1 inputs of every
//    request live in its state slot and are replaced at the end of the step.
//  * ts_group_norm / ts_group_norm_add: RMS norm of every one of `groups` equal consecutive parts
//    of a row, times a weight; written out (optionally only some rows), or added to the 32-bit
//    residual.
//  * ts_axpby: out = a x + b y.
//  * ts_gate_columns: out[t, h * vdim + c] = x[t, h, c] * sigmoid(gate[t, h * vdim + c]) for heads
//    stored wider than their values.
//  * ts_joint_norm_kvwrite: q and k of a token normed over all their heads at once (one weight
//    per column), q to padded rows for the attention kernels, k and v to the token's cache slot.
//  * ts_mlstm_gates: the stabilised gates of a matrix memory with exponential input gate:
//    m_t = max(f_t + m_(t-1), i_t), keep_t = exp(f_t + m_(t-1) - m_t), write_t = exp(i_t - m_t),
//    floor_t = exp(-m_t); i and f capped by cap tanh(. / cap), f through log-sigmoid; m is state.
//  * ts_mlstm_finish: o / (max(|n . q|, floor) + 1e-6), RMS per head, weight, sigmoid gate.
//  * ts_ssm_finish: (y + D x) silu(z), RMS in groups over all heads, weight.
#include "common.cuh"

TS_DEFINE_LAST_ERROR()

namespace {

// an operand that is float or bfloat16, chosen at run time
struct Rows {
  const void* ptr;
  long long ld;
  int is_f32;
  __device__ __forceinline__ float at(size_t row, int col) const {
    return is_f32 ? static_cast<const float*>(ptr)[row * ld + col]
                  : __bfloat162float(static_cast<const __nv_bfloat16*>(ptr)[row * ld + col]);
  }
};
struct RowsOut {
  void* ptr;
  long long ld;
  int is_f32;
  __device__ __forceinline__ void put(size_t row, int col, float v) const {
    if (is_f32) static_cast<float*>(ptr)[row * ld + col] = v;
    else static_cast<__nv_bfloat16*>(ptr)[row * ld + col] = __float2bfloat16_rn(v);
  }
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// ------------------------------------------------------------------ learned positions
__global__ void add_position_rows_kernel(float* __restrict__ residual, VecParam table, const int* __restrict__ positions,
                                         int num_positions, int n) {
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  const int p = positions[t];
  if (p < 0 || p >= num_positions) {
    if (threadIdx.x == 0) ts_raise_status(TS_STATUS_BOUNDS, TS_BAD_POSITION);
    return;
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) residual[t * n + i] += table[(size_t)p * n + i];
}

// ------------------------------------------------------------------ causal convolution over time
constexpr int CONV_TILE = 32;        // tokens of a block
constexpr int CONV_THREADS = 128;    // channels of a block
constexpr int CONV_MAX_TAPS = 8;

struct ConvParams {
  Rows x;
  RowsOut y;
  VecParam w;              // [C, taps]
  VecParam bias;           // [C] or null
  float* state;            // [slots, taps - 1, C]: a request's last inputs, oldest first
  const int* state_slots; const int* fresh; const int* cu_q;
  int C, add_input, silu;
};

// Thread = one channel over CONV_TILE tokens of one request, its last TAPS - 1 inputs in
// registers.  The block of a request's first tile also makes the request's new state: it is the
// only one that reads the old state, so nobody reads what it overwrites.
template <int TAPS>
__global__ void __launch_bounds__(CONV_THREADS) causal_conv_kernel(ConvParams p) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.z;
  const int t0 = p.cu_q[b], n = p.cu_q[b + 1] - t0;
  const int first = blockIdx.y * CONV_TILE;
  const int c = blockIdx.x * CONV_THREADS + threadIdx.x;
  if (first >= n || c >= p.C) return;
  constexpr int H = TAPS - 1;
  float w[TAPS];
#pragma unroll
  for (int j = 0; j < TAPS; ++j) w[j] = p.w[(size_t)c * TAPS + j];
  const float bias = p.bias.ptr ? p.bias[c] : 0.f;
  float* st = p.state + (size_t)p.state_slots[b] * H * p.C + c;
  const bool is_fresh = p.fresh[b] != 0;
  float old[H > 0 ? H : 1];
  if (first < H) {
#pragma unroll
    for (int i = 0; i < H; ++i) old[i] = is_fresh ? 0.f : st[(size_t)i * p.C];
  }
  // hist[i] = input at token first - H + i of this portion (negative tokens: the state)
  float hist[H > 0 ? H : 1];
#pragma unroll
  for (int i = 0; i < H; ++i) {
    const int tok = first - H + i;
    hist[i] = tok >= 0 ? p.x.at(t0 + tok, c) : old[i];      // (tok < 0 only in a request's first tile)
  }
  const int last = min(n, first + CONV_TILE);
  for (int tok = first; tok < last; ++tok) {
    const float cur = p.x.at(t0 + tok, c);
    float acc = bias + w[H] * cur;
#pragma unroll
    for (int i = 0; i < H; ++i) acc = fmaf(w[i], hist[i], acc);
    if (p.silu) acc = silu_f(acc);
    if (p.add_input) acc += cur;
    p.y.put(t0 + tok, c, acc);
#pragma unroll
    for (int i = 0; i + 1 < H; ++i) hist[i] = hist[i + 1];
    if (H > 0) hist[H - 1] = cur;
  }
  if (first == 0) {
    // new state: inputs at tokens n - H .. n - 1 (tokens below 0: the old state, shifted)
#pragma unroll
    for (int i = 0; i < H; ++i) {
      const int tok = n - H + i;
      float v = 0.f;
      if (tok >= 0) v = p.x.at(t0 + tok, c);
      else {
#pragma unroll
        for (int j = 0; j < H; ++j)
          if (j == tok + H) v = old[j];
      }
      st[(size_t)i * p.C] = v;
    }
  }
}

// ------------------------------------------------------------------ RMS norm in groups
// a block per (row, group); y = x / sqrt(mean(x^2) + eps) * w over each group of n / groups.  A thread keeps
// its first ROW_HOLD elements in registers between the sum and the scaling, and reads any further ones twice.
constexpr int ROW_HOLD = 8;

// threads of a block that walks `per` elements of a row: four elements a thread, 32 to 256 threads
inline int row_threads(int per) { return per >= 1024 ? 256 : (per >= 512 ? 128 : (per >= 256 ? 64 : 32)); }

template <bool ADD>
__global__ void group_norm_kernel(Rows x, VecParam w, const int* __restrict__ rows, int groups, int n, float eps,
                                  RowsOut out, float* __restrict__ residual) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const size_t o = blockIdx.x;
  const size_t t = rows ? (size_t)rows[o] : o;
  const int per = n / groups, base = blockIdx.y * per;
  float held[ROW_HOLD], acc = 0.f;
#pragma unroll
  for (int j = 0; j < ROW_HOLD; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    held[j] = i < per ? x.at(t, base + i) : 0.f;
    acc = fmaf(held[j], held[j], acc);
  }
  for (int i = threadIdx.x + ROW_HOLD * blockDim.x; i < per; i += blockDim.x) {
    const float v = x.at(t, base + i);
    acc = fmaf(v, v, acc);
  }
  const float rstd = rsqrtf(block_sum(acc, scratch) / (float)per + eps);
  auto put = [&](int i, float v) {
    const int col = base + i;
    const float y = v * rstd * w[col];
    if (ADD) residual[t * n + col] += y;
    else out.put(o, col, y);
  };
#pragma unroll
  for (int j = 0; j < ROW_HOLD; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < per) put(i, held[j]);
  }
  for (int i = threadIdx.x + ROW_HOLD * blockDim.x; i < per; i += blockDim.x) put(i, x.at(t, base + i));
}

// ------------------------------------------------------------------ a x + b y
__global__ void axpby_kernel(Rows x, Rows y, float a, float b, RowsOut out, long long count) {
  pdl_trigger();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x)
    out.put((size_t)i, 0, a * x.at((size_t)i, 0) + b * y.at((size_t)i, 0));
}

// ------------------------------------------------------------------ heads times an element-wise sigmoid gate
__global__ void gate_columns_kernel(Rows x, Rows gate, RowsOut out, int H, int stored, int vdim) {
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < H * vdim; i += blockDim.x) {
    const int h = i / vdim, c = i % vdim;
    out.put(t, i, x.at(t, h * stored + c) * sigmoid_f(gate.at(t, i)));
  }
}

// ------------------------------------------------------------------ q and k normed over all heads, cache write
struct JointNorm {
  Rows q, k, v;
  VecParam qw, kw;         // [H dim], [G dim]; null: no norm
  float eps;
  int H, G, dim, vdim, stored, page_size;
  void* q_out;             // [T, H, stored]
  void* k_cache; void* v_cache;     // [pages, G, page, stored]
  const int* slot_mapping;          // null: nothing is written
  int out_is_f32;
};

__global__ void joint_norm_kvwrite_kernel(JointNorm p) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  const int nq = p.H * p.dim, nk = p.G * p.dim;
  float aq = 0.f, ak = 0.f;
  if (p.qw.ptr) {
    for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = p.q.at(t, i); aq = fmaf(v, v, aq); }
    for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = p.k.at(t, i); ak = fmaf(v, v, ak); }
  }
  const float rq = p.qw.ptr ? rsqrtf(block_sum(aq, scratch) / (float)nq + p.eps) : 1.f;
  const float rk = p.qw.ptr ? rsqrtf(block_sum(ak, scratch) / (float)nk + p.eps) : 1.f;
  RowsOut qo{p.q_out, (long long)p.H * p.stored, p.out_is_f32};
  for (int i = threadIdx.x; i < p.H * p.stored; i += blockDim.x) {
    const int h = i / p.stored, d = i % p.stored;
    float v = 0.f;
    if (d < p.dim) {
      v = p.q.at(t, h * p.dim + d) * rq;
      if (p.qw.ptr) v *= p.qw[h * p.dim + d];
    }
    qo.put(t, i, v);
  }
  if (!p.slot_mapping) return;
  const int slot = p.slot_mapping[t];
  if (slot < 0) return;
  const size_t page = slot / p.page_size, in_page = slot % p.page_size;
  for (int i = threadIdx.x; i < p.G * p.stored; i += blockDim.x) {
    const int g = i / p.stored, d = i % p.stored;
    float kv = 0.f, vv = 0.f;
    if (d < p.dim) {
      kv = p.k.at(t, g * p.dim + d) * rk;
      if (p.kw.ptr) kv *= p.kw[g * p.dim + d];
    }
    if (d < p.vdim) vv = p.v.at(t, g * p.vdim + d);
    const size_t at = ((page * p.G + g) * p.page_size + in_page) * p.stored + d;
    if (p.out_is_f32) {
      static_cast<float*>(p.k_cache)[at] = kv;
      static_cast<float*>(p.v_cache)[at] = vv;
    } else {
      static_cast<__nv_bfloat16*>(p.k_cache)[at] = __float2bfloat16_rn(kv);
      static_cast<__nv_bfloat16*>(p.v_cache)[at] = __float2bfloat16_rn(vv);
    }
  }
}

// ------------------------------------------------------------------ gates of a matrix memory with exponential input gate
// m_t = max(f_t + m_(t-1), i_t) is a chain of maps x -> max(F + x, I); two such maps compose to another one,
// (F2, I2) o (F1, I1) = (F1 + F2, max(I1 + F2, I2)), so 32 tokens are a warp scan, and a span of tokens has
// one map that can be applied before the span's own maximum is known.
//
// A warp walks the tokens [a, e) of head h 32 at a time.  EMIT: from the maximum m before token a it writes
// keep_t, write_t, exp(-m_t) and returns the maximum after the span in .x.  Otherwise it writes nothing and
// returns the span's map (F, I).
template <bool EMIT>
__device__ __forceinline__ float2 mlstm_gates_walk(const float* __restrict__ raw, long long ld, float cap, int H, int h,
                                                   int a, int e, float m, float* __restrict__ keep,
                                                   float* __restrict__ write, float* __restrict__ floor_) {
  const int lane = threadIdx.x & 31;
  const float inv_cap = 1.f / cap;
  float Fs = 0.f, Is = -INFINITY;
  for (int base = a; base < e; base += 32) {
    const int t = base + lane;
    const bool live = t < e;
    float gi = -INFINITY, gf = 0.f;      // (a lane behind the span holds the identity map)
    if (live) {
      gi = cap * tanhf(raw[(size_t)t * ld + h] * inv_cap);
      gf = log_sigmoid_f(cap * tanhf(raw[(size_t)t * ld + H + h] * inv_cap));
    }
    float F = gf, I = gi;       // the map of tokens base .. t, composed
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float pF = __shfl_up_sync(0xffffffffu, F, o), pI = __shfl_up_sync(0xffffffffu, I, o);
      if (lane >= o) {
        I = fmaxf(pI + F, I);
        F = pF + F;
      }
    }
    if (EMIT) {
      const float m_t = fmaxf(F + m, I);
      float m_prev = __shfl_up_sync(0xffffffffu, m_t, 1);
      if (lane == 0) m_prev = m;
      if (live) {
        keep[(size_t)t * H + h] = expf(gf + m_prev - m_t);
        write[(size_t)t * H + h] = expf(gi - m_t);
        floor_[(size_t)t * H + h] = expf(-m_t);
      }
      m = __shfl_sync(0xffffffffu, m_t, 31);
    } else {
      const float tF = __shfl_sync(0xffffffffu, F, 31), tI = __shfl_sync(0xffffffffu, I, 31);
      Is = fmaxf(Is + tF, tI);
      Fs += tF;
    }
  }
  return EMIT ? make_float2(m, 0.f) : make_float2(Fs, Is);
}

// a warp per (request, head): steps of few tokens a request
__global__ void mlstm_gates_kernel(const float* __restrict__ raw, long long ld, float cap, float* __restrict__ m_state,
                                   const int* __restrict__ state_slots, const int* __restrict__ fresh,
                                   const int* __restrict__ cu_q, int num_requests, int H, float* __restrict__ keep,
                                   float* __restrict__ write, float* __restrict__ floor_) {
  pdl_trigger();
  pdl_wait();
  const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= num_requests * H) return;
  const int b = pair / H, h = pair % H;
  const int t0 = cu_q[b], t1 = cu_q[b + 1];
  if (t1 <= t0) return;
  float* ms = m_state + (size_t)state_slots[b] * H + h;
  const float m = mlstm_gates_walk<true>(raw, ld, cap, H, h, t0, t1, fresh[b] ? 0.f : *ms, keep, write, floor_).x;
  if ((threadIdx.x & 31) == 0) *ms = m;
}

// a block per (request, head): every warp takes a span of the request's tokens, finds the span's map, learns
// the maximum before its span from the maps of the spans before it, and walks its span again to write
__global__ void mlstm_gates_spans_kernel(const float* __restrict__ raw, long long ld, float cap, float* __restrict__ m_state,
                                         const int* __restrict__ state_slots, const int* __restrict__ fresh,
                                         const int* __restrict__ cu_q, int H, float* __restrict__ keep,
                                         float* __restrict__ write, float* __restrict__ floor_) {
  __shared__ float span_f[32], span_i[32];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int b = blockIdx.x / H, h = blockIdx.x % H;
  const int t0 = cu_q[b], t1 = cu_q[b + 1];
  if (t1 <= t0) return;
  float* ms = m_state + (size_t)state_slots[b] * H + h;
  const float m0 = fresh[b] ? 0.f : *ms;
  const int span = (((t1 - t0) + warps - 1) / warps + 31) / 32 * 32;
  const int a = min(t1, t0 + warp * span), e = min(t1, a + span);
  const float2 map = mlstm_gates_walk<false>(raw, ld, cap, H, h, a, e, 0.f, keep, write, floor_);
  if (lane == 0) {
    span_f[warp] = map.x;
    span_i[warp] = map.y;
  }
  __syncthreads();          // (also: every thread has read the old maximum before thread 0 writes the new one)
  float m = m0;
  for (int w = 0; w < warp; ++w) m = fmaxf(span_f[w] + m, span_i[w]);
  mlstm_gates_walk<true>(raw, ld, cap, H, h, a, e, m, keep, write, floor_);
  if (threadIdx.x == 0) {
    float last = m0;
    for (int w = 0; w < warps; ++w) last = fmaxf(span_f[w] + last, span_i[w]);
    *ms = last;
  }
}

// ------------------------------------------------------------------ what follows the scan of a matrix memory
// raw [T, H, wide] 32-bit: columns [0, vdim) the numerator S^T q, column vdim the product n . q
__global__ void mlstm_finish_kernel(const float* __restrict__ raw, int wide, const float* __restrict__ floor_,
                                    VecParam weight, Rows gate, float eps, RowsOut out, int H, int vdim, int num_tokens) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long pair = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= (long long)num_tokens * H) return;
  const size_t t = pair / H;
  const int h = (int)(pair % H);
  const float* o = raw + (t * H + h) * wide;
  const float den = fmaxf(fabsf(o[vdim]), floor_[t * H + h]) + 1e-6f;
  const float inv = 1.f / den;
  float acc = 0.f;
  for (int i = lane; i < vdim; i += 32) {
    const float v = o[i] * inv;
    acc = fmaf(v, v, acc);
  }
  const float rstd = rsqrtf(warp_sum(acc) / (float)vdim + eps);
  for (int i = lane; i < vdim; i += 32) {
    const int col = h * vdim + i;
    float y = o[i] * inv * rstd * weight[col];
    if (gate.ptr) y *= sigmoid_f(gate.at(t, col));
    out.put(t, col, y);
  }
}

// raw [T, H vdim] 32-bit y of the scan; x the scan's values; z the gate; a block per (token, norm group)
__global__ void ssm_finish_kernel(const float* __restrict__ raw, Rows x, VecParam skip, Rows z, VecParam weight, int groups,
                                  float eps, RowsOut out, int H, int vdim) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  const int n = H * vdim, per = n / groups, base = blockIdx.y * per;
  auto gated = [&](int i) {
    const int col = base + i;
    return (raw[t * n + col] + skip[col / vdim] * x.at(t, col)) * silu_f(z.at(t, col));
  };
  float held[ROW_HOLD], acc = 0.f;
#pragma unroll
  for (int j = 0; j < ROW_HOLD; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    held[j] = i < per ? gated(i) : 0.f;
    acc = fmaf(held[j], held[j], acc);
  }
  for (int i = threadIdx.x + ROW_HOLD * blockDim.x; i < per; i += blockDim.x) {
    const float y = gated(i);
    acc = fmaf(y, y, acc);
  }
  const float rstd = rsqrtf(block_sum(acc, scratch) / (float)per + eps);
#pragma unroll
  for (int j = 0; j < ROW_HOLD; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < per) out.put(t, base + i, held[j] * rstd * weight[base + i]);
  }
  for (int i = threadIdx.x + ROW_HOLD * blockDim.x; i < per; i += blockDim.x)
    out.put(t, base + i, gated(i) * rstd * weight[base + i]);
}

}  // namespace

TS_EXPORT int ts_add_position_rows(float* residual, const void* table, int table_is_f32, const int* positions,
                                   int num_positions, int num_tokens, int n, cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && n > 0 && residual && table && positions, "add_position_rows: empty input");
  TS_LAUNCH("add_position_rows", add_position_rows_kernel, num_tokens, n >= 1024 ? 256 : 128, 0, stream, residual,
            VecParam{table, table_is_f32}, positions, num_positions, n);
  return 0;
}

TS_EXPORT int ts_causal_conv_max_taps() { return CONV_MAX_TAPS; }

TS_EXPORT int ts_causal_conv(const void* x, long long ldx, int x_is_f32, void* y, long long ldy, int y_is_f32,
                             const void* w, int w_is_f32, const void* bias, int taps, float* state, const int* state_slots,
                             const int* fresh, const int* cu_q, int num_requests, int max_q_len, int C, int add_input,
                             int silu, cudaStream_t stream) {
  TS_REQUIRE(num_requests > 0 && max_q_len > 0 && C > 0, "causal_conv: empty input");
  TS_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS, "causal_conv: 1 to %d taps, got %d", CONV_MAX_TAPS, taps);
  TS_REQUIRE(x && y && w && (taps == 1 || state) && state_slots && fresh && cu_q, "causal_conv: a null operand");
  ConvParams p{Rows{x, ldx, x_is_f32}, RowsOut{y, ldy, y_is_f32}, VecParam{w, w_is_f32}, VecParam{bias, w_is_f32},
               state, state_slots, fresh, cu_q, C, add_input, silu};
  const dim3 grid((C + CONV_THREADS - 1) / CONV_THREADS, (max_q_len + CONV_TILE - 1) / CONV_TILE, num_requests);
  TS_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "causal_conv: the step is too large");
  switch (taps) {
#define TS_CONV_CASE(N) \
    case N: TS_LAUNCH("causal_conv", causal_conv_kernel<N>, grid, CONV_THREADS, 0, stream, p); break;
    TS_CONV_CASE(1) TS_CONV_CASE(2) TS_CONV_CASE(3) TS_CONV_CASE(4) TS_CONV_CASE(5) TS_CONV_CASE(6) TS_CONV_CASE(7)
    TS_CONV_CASE(8)
#undef TS_CONV_CASE
  }
  return 0;
}

// rows null: every row of x [num_out, n]; else out[o] = norm(x[rows[o]])
TS_EXPORT int ts_group_norm(const void* x, long long ldx, int x_is_f32, const void* w, int w_is_f32, const int* rows,
                            int groups, int n, float eps, void* out, int out_is_f32, int num_out, cudaStream_t stream) {
  TS_REQUIRE(num_out > 0 && n > 0 && groups > 0 && groups <= 65535 && n % groups == 0, "group_norm: %d columns in %d groups", n, groups);
  TS_LAUNCH("group_norm", group_norm_kernel<false>, dim3(num_out, groups), row_threads(n / groups), 0, stream, Rows{x, ldx, x_is_f32},
            VecParam{w, w_is_f32}, rows, groups, n, eps, RowsOut{out, (long long)n, out_is_f32}, (float*)nullptr);
  return 0;
}

// residual [T, n] (float, in place) += norm(y)
TS_EXPORT int ts_group_norm_add(const void* y, long long ldy, int y_is_f32, const void* w, int w_is_f32, int groups, int n,
                                float eps, float* residual, int num_tokens, cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && n > 0 && groups > 0 && groups <= 65535 && n % groups == 0, "group_norm_add: %d columns in %d groups", n, groups);
  TS_LAUNCH("group_norm_add", group_norm_kernel<true>, dim3(num_tokens, groups), row_threads(n / groups), 0, stream, Rows{y, ldy, y_is_f32},
            VecParam{w, w_is_f32}, (const int*)nullptr, groups, n, eps, RowsOut{nullptr, 0, 0}, residual);
  return 0;
}

TS_EXPORT int ts_axpby(const void* x, const void* y, int in_is_f32, float a, float b, void* out, int out_is_f32,
                       long long count, cudaStream_t stream) {
  TS_REQUIRE(count > 0 && x && y && out, "axpby: empty input");
  const int blocks = (int)((count + 255) / 256 < 148 * 16 ? (count + 255) / 256 : 148 * 16);
  TS_LAUNCH("axpby", axpby_kernel, blocks, 256, 0, stream, Rows{x, 1, in_is_f32}, Rows{y, 1, in_is_f32}, a, b,
            RowsOut{out, 1, out_is_f32}, count);
  return 0;
}

TS_EXPORT int ts_gate_columns(const void* x, const void* gate, long long ldg, int is_f32, void* out, int H, int stored,
                              int vdim, int num_tokens, cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && H > 0 && vdim > 0 && stored >= vdim && x && gate && out, "gate_columns: operands do not fit");
  TS_LAUNCH("gate_columns", gate_columns_kernel, num_tokens, H * vdim >= 2048 ? 512 : (H * vdim >= 1024 ? 256 : 128), 0, stream,
            Rows{x, (long long)H * stored, is_f32}, Rows{gate, ldg, is_f32}, RowsOut{out, (long long)H * vdim, is_f32}, H, stored,
            vdim);
  return 0;
}

TS_EXPORT int ts_joint_norm_kvwrite(int is_f32, const void* q, long long ldq, const void* k, long long ldk, const void* v,
                                    long long ldv, const void* qw, const void* kw, int w_is_f32, float eps, int H, int G,
                                    int dim, int vdim, int stored, void* q_out, void* k_cache, void* v_cache,
                                    const int* slot_mapping, int page_size, int num_tokens, cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && H > 0 && G > 0 && dim > 0 && vdim > 0 && stored >= dim && stored >= vdim,
             "joint_norm_kvwrite: sizes do not fit");
  TS_REQUIRE((qw == nullptr) == (kw == nullptr), "joint_norm_kvwrite: q and k are normed together or not at all");
  TS_REQUIRE(slot_mapping == nullptr || (k_cache && v_cache && page_size > 0), "joint_norm_kvwrite: no cache to write");
  JointNorm p{Rows{q, ldq, is_f32}, Rows{k, ldk, is_f32}, Rows{v, ldv, is_f32}, VecParam{qw, w_is_f32},
              VecParam{kw, w_is_f32}, eps, H, G, dim, vdim, stored, page_size, q_out, k_cache, v_cache, slot_mapping, is_f32};
  TS_LAUNCH("joint_norm_kvwrite", joint_norm_kvwrite_kernel, num_tokens, H * dim >= 2048 ? 512 : (H * dim >= 512 ? 256 : 128), 0, stream, p);
  return 0;
}

TS_EXPORT int ts_mlstm_gates(const float* raw, long long ld, float cap, float* m_state, const int* state_slots,
                             const int* fresh, const int* cu_q, int num_requests, int max_q_len, int H, float* keep,
                             float* write, float* floor_, cudaStream_t stream) {
  TS_REQUIRE(num_requests > 0 && H > 0 && cap > 0.f, "mlstm_gates: empty input or a cap that is not positive");
  TS_REQUIRE(raw && m_state && state_slots && fresh && cu_q && keep && write && floor_, "mlstm_gates: a null operand");
  if (max_q_len >= 128) {
    const int warps = max_q_len >= 512 ? 16 : (max_q_len + 31) / 32;
    TS_LAUNCH("mlstm_gates", mlstm_gates_spans_kernel, num_requests * H, warps * 32, 0, stream, raw, ld, cap, m_state,
              state_slots, fresh, cu_q, H, keep, write, floor_);
    return 0;
  }
  const int warps = 4;
  TS_LAUNCH("mlstm_gates", mlstm_gates_kernel, (num_requests * H + warps - 1) / warps, warps * 32, 0, stream, raw, ld, cap,
            m_state, state_slots, fresh, cu_q, num_requests, H, keep, write, floor_);
  return 0;
}

TS_EXPORT int ts_mlstm_finish(const float* raw, int wide, const float* floor_, const void* weight, int w_is_f32,
                              const void* gate, long long ldg, int io_is_f32, float eps, void* out, int H, int vdim,
                              int num_tokens, cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && H > 0 && vdim > 0 && wide > vdim && raw && floor_ && weight && out,
             "mlstm_finish: operands do not fit");
  const int warps = 4;
  const long long pairs = (long long)num_tokens * H;
  TS_LAUNCH("mlstm_finish", mlstm_finish_kernel, (int)((pairs + warps - 1) / warps), warps * 32, 0, stream, raw, wide,
            floor_, VecParam{weight, w_is_f32}, Rows{gate, ldg, io_is_f32}, eps,
            RowsOut{out, (long long)H * vdim, io_is_f32}, H, vdim, num_tokens);
  return 0;
}

TS_EXPORT int ts_ssm_finish(const float* raw, const void* x, long long ldx, const void* skip, const void* z, long long ldz,
                            const void* weight, int w_is_f32, int io_is_f32, int groups, float eps, void* out, int H,
                            int vdim, int num_tokens, cudaStream_t stream) {
  TS_REQUIRE(num_tokens > 0 && H > 0 && vdim > 0 && groups > 0 && groups <= 65535 && (H * vdim) % groups == 0,
             "ssm_finish: %d columns in %d groups", H * vdim, groups);
  TS_REQUIRE(raw && x && skip && z && weight && out, "ssm_finish: a null operand");
  TS_LAUNCH("ssm_finish", ssm_finish_kernel, dim3(num_tokens, groups), row_threads(H * vdim / groups), 0, stream, raw, Rows{x, ldx, io_is_f32},
            VecParam{skip, w_is_f32}, Rows{z, ldz, io_is_f32}, VecParam{weight, w_is_f32}, groups, eps,
            RowsOut{out, (long long)H * vdim, io_is_f32}, H, vdim);
  return 0;
}
