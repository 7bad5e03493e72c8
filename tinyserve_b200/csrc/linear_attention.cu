// Linear attention with a decaying matrix state, for one key size per build (-DTS_KEY_DIM=...):
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T        (S: key size x value size, per request and head)
//   o_t = S_t^T q_t
//
// a_t is one constant per head (retention: `decay`), or one number per key channel and token made
// from 32-bit logits z (gated linear attention: a_t = sigmoid(z_t)^(1 / tau); with a lower bound l per
// channel a_t = l + (1 - l) sigmoid(z_t), and then k_t may be tied to it, k_t = 1 - a_t), or one
// number per head and token that the caller made (`tok_keep`, with a factor `tok_write` on k_t:
// S_t = keep_t S_(t-1) + write_t k_t v_t^T, the form of selective state spaces and of matrix
// memories with an exponential input gate; for a selective state space the kernel may make both itself
// from the 32-bit step-size logits: dt = softplus(raw + bias_h), keep = exp(-exp(rate_h) dt), write = dt).  Several heads may share one q and k (`qk_group`).
// The values may get constant columns behind the ones the caller brings (`v_width` < value size: a
// column of ones, then zeros), so that S^T q also holds sum_t (...) k_t . q, a normaliser.
// q and k may get rotary positions on their first rotary_dim elements and a constant factor
// each.  The head's output is divided by its root mean square over the value size (times an
// optional weight), multiplied by silu(gate) and stored as T for the output projection.
//
// The state is 32-bit, lives in the request's state slot between steps, and starts at zero for
// a request whose first token is in this step.  Everything after the projections is 32-bit
// arithmetic: angles, decays, the state, the output norm.  T is the storage type of the
// projections, the gate and the result (float or bfloat16).
//
// One block per (request, head) walks the request's tokens of this step in order, a single
// decoded token and a prompt portion of any length alike.  (A head with more value columns than
// a block takes is spread over several blocks; the output norm, which needs the whole head, then
// runs as a kernel of its own on the 32-bit outputs.)  A thread keeps a tile of up to 16 rows x 4
// columns of the state in registers; the row groups of a column quad are neighbouring lanes and
// add their shares of o_t by shuffles.  Tokens are staged through shared memory sixteen at a
// time (rotary, factors and decays applied while staging), and the output norm and gate run
// once per sixteen tokens on the staged outputs.
//
// Long portions are cut into segments of `seg_len` tokens that run side by side (a request of
// 2,048 tokens and 8 heads alone would keep 8 of 148 SMs busy): the recurrence is linear in S, so
//   (1) every segment but a request's last runs from a zero state and leaves its local end state
//       L_p and the product D_p of its decays (SCAN_LOCAL),
//   (2) one pass over the segments turns them into start states, S_(p+1) = D_p S_p + L_p, from
//       the request's stored state (combine kernel),
//   (3) every segment runs again from its start state and makes its outputs; the last one stores
//       the request's new state (SCAN_FROM_SEGMENT).
// Nothing is divided by a decay anywhere, so no product of decays can overflow or vanish into a
// division.  Short portions and decoded tokens run as one segment in one launch (SCAN_WHOLE).
#include "common.cuh"

#ifndef TS_KEY_DIM
#error "compile with -DTS_KEY_DIM=<key size>"
#endif

TS_DEFINE_LAST_ERROR()

namespace {

constexpr int DIM = TS_KEY_DIM;
// Row groups of a column: the smallest power of two that divides the key size and leaves a
// thread at most 16 state rows (a thread keeps rows x COLS state elements in registers); key
// sizes that no power of two cuts that small get up to 32, then up to 64 rows a thread.
constexpr int pick_groups() {
  for (int most = 16; most <= 64; most *= 2)
    for (int g = 1; g <= 32; g *= 2)
      if (DIM % g == 0 && DIM / g <= most) return g;
  return 0;
}
constexpr int GROUPS = pick_groups();
static_assert(GROUPS > 0, "the key size must split into 1, 2, 4, ... 32 groups of at most 64 rows");
constexpr int R = DIM / GROUPS;           // state rows of a thread
constexpr int COLS = 4;                   // state columns of a thread
constexpr int RP = (R + 3) / 4 * 4 + 4;   // padded length of a group's run in shared memory (16-byte runs, spread over banks)
constexpr int CHUNK = 16;                 // tokens staged at a time
constexpr int MAX_THREADS = 512;
#ifndef TS_SCAN_BLOCKS
#define TS_SCAN_BLOCKS 1                  // blocks per SM that the register count is held to
#endif
constexpr int MAX_COLS = 256;             // value columns of a block at most (a whole head, where it fits)

struct ScanParams {
  const void* q; const void* k; const void* v; const void* gate;
  long long ldq, ldk, ldv, ldg;           // row strides in elements
  const float* z; long long ldz;          // per-channel decay logits [T, H * DIM], or null
  const float* decay;                     // [H], used when z and tok_keep are null
  float inv_tau;
  const int* positions; const float* cos; const float* sin; int rotary_dim;
  float q_scale, k_scale;
  float* state;                           // [slots, H, DIM, vdim]
  const int* state_slots; const int* fresh; const int* cu_q;
  const void* norm_weight; int norm_weight_is_f32; float eps;
  void* out; long long ldo;               // [T, H * vdim]
  int H, vdim;
  int seg_len;                            // tokens per segment; 0: a request's tokens are one segment
  float* seg_state;                       // [B, H, segments, DIM, vdim]: local end states, then start states
  float* seg_decay;                       // [B, H, segments, DIM]: product of a segment's decays (per channel)
  int max_segments;
  int cols, col_tiles;                    // value columns per block (a multiple of COLS); blocks per head
  float* raw_out;                         // [T, H * vdim] 32-bit o_t before norm and gate (col_tiles > 1 or joint_norm), else null
  int in_act;                             // bits ACT_Q, ACT_K, ACT_V: that operand passes through silu as it is staged
  int gate_act;                           // 0: the output is multiplied by silu(gate), 1: by sigmoid(gate)
  int joint_norm;                         // 1: the output norm runs over all heads of a token together (weight [H * vdim])
  const float* lower;                     // [H * DIM] or null: a = lower + (1 - lower) sigmoid(z)
  int tied_key;                           // 1: k = 1 - a (per-channel decays only; `k` is not read)
  const float* tok_keep;                  // [T, H] or null: the decay of (token, head)
  const float* tok_write;                 // [T, H]: factor on k of (token, head)
  int qk_group;                           // heads that share one q and one k (1: every head its own)
  int v_width;                            // value columns the caller brings per head; behind them a column of ones, then zeros
  int finish;                             // 0: the 32-bit outputs in raw_out are all the caller wants
  const float* step_raw; long long ld_step;   // [T, H] or null: step-size logits, in place of tok_keep / tok_write
  VecParam step_bias, step_rate;              // [H] each: dt = softplus(raw + bias), keep = exp(-exp(rate) dt), write = dt
};

enum { DECAY_HEAD = 0, DECAY_CHANNEL = 1, DECAY_TOKEN = 2 };
enum { ACT_Q = 1, ACT_K = 2, ACT_V = 4 };

__device__ __forceinline__ float staged(float x, int in_act) { return in_act ? x / (1.f + expf(-x)) : x; }
__device__ __forceinline__ float gate_factor(float g, int gate_act) {
  const float s = 1.f / (1.f + expf(-g));
  return gate_act ? s : g * s;
}

enum { SCAN_WHOLE = 0, SCAN_LOCAL = 1, SCAN_FROM_SEGMENT = 2 };

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float softplus(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// Ask for the 128-byte lines of `rows` runs of `bytes` bytes, `stride` bytes apart, to be brought
// into L1: the staging of the next chunk then finds its operands there instead of waiting for L2
// or HBM behind a barrier.  A hint only: nothing is read into registers and nothing waits.
__device__ __forceinline__ void prefetch_rows(const void* first, long long stride, int bytes, int rows, int warp, int warps,
                                              int lane) {
  const char* base = static_cast<const char*>(first);
  for (int row = warp; row < rows; row += warps)
    for (int at = lane * 128; at < bytes + 127; at += 32 * 128) {       // (a run that starts inside a line touches one more)
      const char* ptr = base + (long long)row * stride + (at < bytes ? at : bytes - 1);
      asm volatile("prefetch.global.L1 [%0];" ::"l"(ptr));
    }
}

// Thread (column quad lc, row group g) keeps rows [g R, (g + 1) R) of columns [4 lc, 4 lc + 4) of
// the block's columns: per token it reads R values each of q, k (and the decays) and four of v
// from shared memory for 3 R x 4 multiply-adds, so the arithmetic, not shared memory, is what
// it waits for.  The row groups of a column quad are neighbouring lanes and add their shares of
// o_t by shuffles.
template <typename T, int DECAY, int MODE>
__global__ void __launch_bounds__(MAX_THREADS, TS_SCAN_BLOCKS) linear_attention_scan_kernel(ScanParams p) {
  constexpr bool PER_CHANNEL = DECAY == DECAY_CHANNEL;
  extern __shared__ float smem[];
  __shared__ float s_keep[CHUNK];                     // DECAY_TOKEN: the staged tokens' decays
  const int vdim = p.vdim, cols = p.cols;
  float* sq = smem;                                   // [CHUNK][GROUPS][RP]
  float* sk = sq + CHUNK * GROUPS * RP;
  float* sa = sk + CHUNK * GROUPS * RP;               // PER_CHANNEL only
  float* sv = sa + (PER_CHANNEL ? CHUNK * GROUPS * RP : 0);   // [CHUNK][cols]
  float* so = sv + CHUNK * cols;                      // [CHUNK][cols]
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x / p.col_tiles, col0 = (blockIdx.x % p.col_tiles) * cols, h = blockIdx.y, seg = blockIdx.z;
  int t0 = p.cu_q[b], t1 = p.cu_q[b + 1];
  const int request_end = t1;
  if (MODE != SCAN_WHOLE) {
    t0 += seg * p.seg_len;
    t1 = min(t1, t0 + p.seg_len);
  }
  if (t1 <= t0) return;
  const bool last = t1 == request_end;
  if (MODE == SCAN_LOCAL && last) return;          // the last segment's end state is the output pass's
  const int tid = threadIdx.x, lc = tid / GROUPS, g = tid % GROUPS;
  const int c = col0 + lc * COLS;                  // first of the thread's columns in the head
  const bool in_block = lc * COLS < cols;
  bool owns[COLS];
#pragma unroll
  for (int j = 0; j < COLS; ++j) owns[j] = in_block && c + j < vdim;
  const bool quad = owns[COLS - 1] && vdim % 4 == 0;        // four columns, 16-byte aligned in every row
  const int slot = p.state_slots[b];
  float* S = p.state + (((size_t)slot * p.H + h) * DIM + (size_t)g * R) * vdim + c;
  const size_t seg_index = ((size_t)b * p.H + h) * p.max_segments + seg;
  float* seg_S = MODE == SCAN_WHOLE ? nullptr : p.seg_state + (seg_index * DIM + (size_t)g * R) * vdim + c;
  float s[R][COLS];
  float w[PER_CHANNEL && MODE == SCAN_LOCAL ? R : 1];      // local pass: product of the decays behind the current token
#pragma unroll
  for (int r = 0; r < (PER_CHANNEL && MODE == SCAN_LOCAL ? R : 1); ++r) w[r] = 1.f;
  const float* from = MODE == SCAN_WHOLE ? (p.fresh[b] ? nullptr : S) : (MODE == SCAN_FROM_SEGMENT ? seg_S : nullptr);
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (from && quad) {
      const float4 x = *reinterpret_cast<const float4*>(from + (size_t)r * vdim);
      s[r][0] = x.x; s[r][1] = x.y; s[r][2] = x.z; s[r][3] = x.w;
    } else {
#pragma unroll
      for (int j = 0; j < COLS; ++j) s[r][j] = from && owns[j] ? from[(size_t)r * vdim + j] : 0.f;
    }
  }
  const float head_decay = DECAY == DECAY_HEAD ? p.decay[h] : 1.f;
  const int hq = h / p.qk_group, vw = p.v_width;
  const bool tied = PER_CHANNEL && p.tied_key;
  const int act_q = p.in_act & ACT_Q, act_k = p.in_act & ACT_K, act_v = p.in_act & ACT_V;
  const T* q = static_cast<const T*>(p.q) + (size_t)hq * DIM;
  const T* k = static_cast<const T*>(p.k) + (size_t)hq * DIM;
  const T* v = static_cast<const T*>(p.v) + (size_t)h * vw;
  const T* gate = static_cast<const T*>(p.gate) + (size_t)h * vdim;
  T* out = static_cast<T*>(p.out) + (size_t)h * vdim;
  const int rot = p.rotary_dim, half = rot >> 1;
  VecParam nw{p.norm_weight, p.norm_weight_is_f32};
  const int warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;

  // The local pass walks its segment backwards: with w_t the product of the decays behind token t,
  // the end state from zero is sum_t (w_t k_t) v_t^T, one multiply-add per state element and token
  // (the recurrence costs two), and w ends as the product of all the segment's decays.
  const int chunks = (t1 - t0 + CHUNK - 1) / CHUNK;
  for (int turn = 0; turn < chunks; ++turn) {
    const int base = t0 + (MODE == SCAN_LOCAL ? chunks - 1 - turn : turn) * CHUNK;
    const int next = MODE == SCAN_LOCAL ? base - CHUNK : base + CHUNK;
    const int n = min(CHUNK, t1 - base);
    // stage q, k (rotary and factor applied), the decays and v.  The loads are read-only ones
    // (what they read was finished before this kernel's wait returned), several in flight per
    // thread: a chunk's staging would otherwise cost as much as its arithmetic
    // (a warp per token, lanes along the row: no division by a run-time length anywhere)
    auto where = [](int tok, int i) { return (tok * GROUPS + i / R) * RP + i % R; };
    for (int tok = warp; tok < n; tok += warps) {
      const size_t t = base + tok;
      const T* kt = k + t * p.ldk;
      const T* qt = q + t * p.ldq;
      float k_factor = p.k_scale;
      if (DECAY == DECAY_TOKEN) {
        if (p.step_raw) {
          const float dt = softplus(__ldg(p.step_raw + t * p.ld_step + h) + p.step_bias[h]);
          k_factor *= dt;
          if (lane == 0) s_keep[tok] = expf(-expf(p.step_rate[h]) * dt);
        } else {
          k_factor *= __ldg(p.tok_write + t * p.H + h);
          if (lane == 0) s_keep[tok] = __ldg(p.tok_keep + t * p.H + h);
        }
      }
      if (half > 0) {
        const size_t at = (size_t)__ldg(p.positions + t) * half;
#pragma unroll 2
        for (int j = lane; j < half; j += 32) {                    // a pair (j, j + half) per turn
          const float cs = __ldg(p.cos + at + j), sn = __ldg(p.sin + at + j);
          const float ka = staged(to_f32<T>(__ldg(kt + j)), act_k), kb = staged(to_f32<T>(__ldg(kt + j + half)), act_k);
          sk[where(tok, j)] = (ka * cs - kb * sn) * k_factor;
          sk[where(tok, j + half)] = (kb * cs + ka * sn) * k_factor;
          if (MODE != SCAN_LOCAL) {
            const float qa = staged(to_f32<T>(__ldg(qt + j)), act_q), qb = staged(to_f32<T>(__ldg(qt + j + half)), act_q);
            sq[where(tok, j)] = (qa * cs - qb * sn) * p.q_scale;
            sq[where(tok, j + half)] = (qb * cs + qa * sn) * p.q_scale;
          }
        }
      }
#pragma unroll 2
      for (int i = rot + lane; i < DIM; i += 32) {                 // the elements behind the rotary ones
        if (!tied) sk[where(tok, i)] = staged(to_f32<T>(__ldg(kt + i)), act_k) * k_factor;
        if (MODE != SCAN_LOCAL) sq[where(tok, i)] = staged(to_f32<T>(__ldg(qt + i)), act_q) * p.q_scale;
      }
      if (PER_CHANNEL) {
        const float* zt = p.z + t * p.ldz + (size_t)h * DIM;
        const float* low = p.lower ? p.lower + (size_t)h * DIM : nullptr;
#pragma unroll 2
        for (int i = lane; i < DIM; i += 32) {
          float a, rest;      // rest = 1 - a, made without the cancellation of that difference
          if (low) {
            const float l = __ldg(low + i), zz = __ldg(zt + i);
            a = l + (1.f - l) / (1.f + expf(-zz));
            rest = (1.f - l) / (1.f + expf(zz));
          } else {
            a = expf(log_sigmoid(__ldg(zt + i)) * p.inv_tau);
            rest = 1.f - a;
          }
          sa[where(tok, i)] = a;
          if (tied) sk[where(tok, i)] = rest * k_factor;
        }
      }
      const T* vt = v + t * p.ldv + col0;
#pragma unroll 4
      for (int i = lane; i < cols; i += 32)
        sv[tok * cols + i] = col0 + i < vw ? staged(to_f32<T>(__ldg(vt + i)), act_v) : (col0 + i == vw && vw < vdim ? 1.f : 0.f);
    }
    __syncthreads();
    if (turn + 1 < chunks) {        // the next chunk's operands, on their way while this one is computed
      const int m = min(CHUNK, t1 - next);
      const size_t t = next;
      if (!tied) prefetch_rows(k + t * p.ldk, p.ldk * (long long)sizeof(T), DIM * (int)sizeof(T), m, warp, warps, lane);
      if (col0 < vw)
        prefetch_rows(v + t * p.ldv + col0, p.ldv * (long long)sizeof(T), min(cols, vw - col0) * (int)sizeof(T), m, warp, warps, lane);
      if (PER_CHANNEL) prefetch_rows(p.z + t * p.ldz + (size_t)h * DIM, p.ldz * 4, DIM * 4, m, warp, warps, lane);
      if (MODE != SCAN_LOCAL) {
        prefetch_rows(q + t * p.ldq, p.ldq * (long long)sizeof(T), DIM * (int)sizeof(T), m, warp, warps, lane);
        if (p.gate && !p.raw_out)
          prefetch_rows(gate + t * p.ldg, p.ldg * (long long)sizeof(T), vdim * (int)sizeof(T), m, warp, warps, lane);
      }
      if (half > 0) {
        const size_t at = (size_t)__ldg(p.positions + t) * half;          // (a request's positions in a step are consecutive)
        prefetch_rows(p.cos + at, half * 4, half * 4, m, warp, warps, lane);
        prefetch_rows(p.sin + at, half * 4, half * 4, m, warp, warps, lane);
      }
    }
    if (in_block) {       // (whole warps or none: cols is a multiple of 32 / GROUPS columns quads, see the launch)
      if constexpr (MODE == SCAN_LOCAL) {
        for (int tok = n - 1; tok >= 0; --tok) {
          const float* kr = sk + (tok * GROUPS + g) * RP;
          const float* ar = sa + (tok * GROUPS + g) * RP;
          const float4 v4 = *reinterpret_cast<const float4*>(sv + tok * cols + lc * COLS);
          const float vv[COLS] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const float kw = kr[r] * (PER_CHANNEL ? w[r] : w[0]);
#pragma unroll
            for (int j = 0; j < COLS; ++j) s[r][j] = fmaf(kw, vv[j], s[r][j]);
            if (PER_CHANNEL) w[r] *= ar[r];
          }
          if (!PER_CHANNEL) w[0] *= DECAY == DECAY_TOKEN ? s_keep[tok] : head_decay;
        }
      } else
      for (int tok = 0; tok < n; ++tok) {
        const float* qr = sq + (tok * GROUPS + g) * RP;
        const float* kr = sk + (tok * GROUPS + g) * RP;
        const float* ar = sa + (tok * GROUPS + g) * RP;
        const float4 v4 = *reinterpret_cast<const float4*>(sv + tok * cols + lc * COLS);
        const float vv[COLS] = {v4.x, v4.y, v4.z, v4.w};
        float acc[COLS] = {0.f, 0.f, 0.f, 0.f};
        const float token_decay = DECAY == DECAY_TOKEN ? s_keep[tok] : head_decay;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float a = PER_CHANNEL ? ar[r] : token_decay;
          const float kk = kr[r], qq = qr[r];
#pragma unroll
          for (int j = 0; j < COLS; ++j) {
            s[r][j] = fmaf(a, s[r][j], kk * vv[j]);
            acc[j] = fmaf(s[r][j], qq, acc[j]);
          }
        }
#pragma unroll
        for (int o = 1; o < GROUPS; o <<= 1) {
#pragma unroll
          for (int j = 0; j < COLS; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
        }
        if (g == 0) *reinterpret_cast<float4*>(so + tok * cols + lc * COLS) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      }
    }
    __syncthreads();
    // output norm over the value size, gate, store: a warp per token
    if constexpr (MODE != SCAN_LOCAL)
    for (int tok = warp; tok < n; tok += warps) {
      const size_t t = base + tok;
      if (p.raw_out) {            // the head spans several blocks: its norm is another kernel's
        for (int i = lane; i < cols && col0 + i < vdim; i += 32)
          p.raw_out[t * p.H * vdim + (size_t)h * vdim + col0 + i] = so[tok * cols + i];
        continue;
      }
      float acc = 0.f;
      for (int i = lane; i < vdim; i += 32) acc += so[tok * cols + i] * so[tok * cols + i];
      const float rstd = rsqrtf(warp_sum(acc) / (float)vdim + p.eps);
      for (int i = lane; i < vdim; i += 32) {
        float o = so[tok * cols + i] * rstd;
        if (p.norm_weight) o *= nw[i];
        if (p.gate) {
          o *= gate_factor(to_f32<T>(gate[t * p.ldg + i]), p.gate_act);
        }
        out[t * p.ldo + i] = from_f32<T>(o);
      }
    }
    if constexpr (MODE != SCAN_LOCAL) __syncthreads();
  }
  float* to = MODE == SCAN_LOCAL ? seg_S : ((MODE == SCAN_WHOLE || last) ? S : nullptr);
  if (to) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (quad) {
        *reinterpret_cast<float4*>(to + (size_t)r * vdim) = make_float4(s[r][0], s[r][1], s[r][2], s[r][3]);
      } else {
#pragma unroll
        for (int j = 0; j < COLS; ++j)
          if (owns[j]) to[(size_t)r * vdim + j] = s[r][j];
      }
    }
  }
  if (DECAY != DECAY_HEAD && MODE == SCAN_LOCAL && c == 0 && in_block) {     // (per token: the same product for every row)
#pragma unroll
    for (int r = 0; r < R; ++r) p.seg_decay[seg_index * DIM + g * R + r] = w[PER_CHANNEL && MODE == SCAN_LOCAL ? r : 0];
  }
}

// o_t of whole heads (32-bit) -> o / rms(o) (* weight) * silu(gate), stored as T: a warp per
// (token, head), for heads that the scan spread over several blocks
template <typename T>
__global__ void linear_attention_finish_kernel(ScanParams p, int num_tokens) {
  pdl_trigger();
  pdl_wait();
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t t = blockIdx.x;
  const int vdim = p.vdim;
  VecParam nw{p.norm_weight, p.norm_weight_is_f32};
  if (p.joint_norm) {           // one norm over all heads of the token
    __shared__ float scratch[33];
    const int n = p.H * vdim;
    const float* o = p.raw_out + t * n;
    float acc = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) acc += o[i] * o[i];
    const float rstd = rsqrtf(block_sum(acc, scratch) / (float)n + p.eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float y = o[i] * rstd;
      if (p.norm_weight) y *= nw[i];
      if (p.gate) y *= gate_factor(to_f32<T>(static_cast<const T*>(p.gate)[t * p.ldg + i]), p.gate_act);
      static_cast<T*>(p.out)[t * p.ldo + i] = from_f32<T>(y);
    }
    return;
  }
  for (int h = warp; h < p.H; h += warps) {
    const float* o = p.raw_out + t * p.H * vdim + (size_t)h * vdim;
    float acc = 0.f;
    for (int i = lane; i < vdim; i += 32) acc += o[i] * o[i];
    const float rstd = rsqrtf(warp_sum(acc) / (float)vdim + p.eps);
    for (int i = lane; i < vdim; i += 32) {
      float y = o[i] * rstd;
      if (p.norm_weight) y *= nw[i];
      if (p.gate) {
        y *= gate_factor(to_f32<T>(static_cast<const T*>(p.gate)[t * p.ldg + (size_t)h * vdim + i]), p.gate_act);
      }
      static_cast<T*>(p.out)[t * p.ldo + (size_t)h * vdim + i] = from_f32<T>(y);
    }
  }
}

// Local end states -> start states, in place: one thread per state element walks its request's
// segments in order.  Segment 0 starts from the request's stored state (zero for a request that
// starts); S_(p+1) = D_p S_p + L_p with D_p the product of segment p's decays (per head: the
// decay multiplied seg_len times, as the scan itself does).
template <int DECAY>
__global__ void linear_attention_combine_kernel(ScanParams p) {
  constexpr bool PER_CHANNEL = DECAY != DECAY_HEAD;     // a stored product per (segment, row)
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y;
  const int n = p.cu_q[b + 1] - p.cu_q[b];
  const int segments = (n + p.seg_len - 1) / p.seg_len;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;
  if (segments <= 0 || e >= DIM * p.vdim) return;
  const int row = e / p.vdim;
  float s = p.fresh[b] ? 0.f : p.state[((size_t)p.state_slots[b] * p.H + h) * DIM * p.vdim + e];
  float head_decay = 1.f;
  if (!PER_CHANNEL) {
    const float d = p.decay[h];
    for (int i = 0; i < p.seg_len; ++i) head_decay *= d;
  }
  const size_t first = ((size_t)b * p.H + h) * p.max_segments;
  // eight segments' loads at a time, then their chain of multiply-adds: the loads do not wait for one another
  constexpr int BATCH = 8;
  for (int seg0 = 0; seg0 < segments; seg0 += BATCH) {
    float local[BATCH], d[BATCH];
#pragma unroll
    for (int j = 0; j < BATCH; ++j) {
      const int seg = seg0 + j;
      const bool inner = seg + 1 < segments;       // (the last segment left no local state: the output pass makes the request's new one)
      local[j] = inner ? p.seg_state[(first + seg) * DIM * p.vdim + e] : 0.f;
      d[j] = PER_CHANNEL ? (inner ? p.seg_decay[(first + seg) * DIM + row] : 0.f) : head_decay;
    }
#pragma unroll
    for (int j = 0; j < BATCH; ++j) {
      if (seg0 + j < segments) p.seg_state[(first + seg0 + j) * DIM * p.vdim + e] = s;
      s = fmaf(d[j], s, local[j]);
    }
  }
}

template <typename T, int DECAY, int MODE>
int launch_scan_mode(const ScanParams& p, int num_requests, int segments, cudaStream_t stream) {
  const int threads = p.cols / COLS * GROUPS;       // a multiple of 32: see the choice of cols
  constexpr bool PER_CHANNEL = DECAY == DECAY_CHANNEL;
  const size_t smem = ((size_t)(PER_CHANNEL ? 3 : 2) * CHUNK * GROUPS * RP + 2 * (size_t)CHUNK * p.cols) * sizeof(float);
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(linear_attention_scan_kernel<T, DECAY, MODE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ts_fail("linear_attention: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    allowed = smem;
  }
  TS_LAUNCH("linear_attention", (linear_attention_scan_kernel<T, DECAY, MODE>),
            dim3(num_requests * p.col_tiles, p.H, segments), threads, smem, stream, p);
  return 0;
}

template <typename T, int DECAY>
int launch_scan(const ScanParams& p, int num_requests, int num_tokens, cudaStream_t stream) {
  if (p.seg_len <= 0) {
    if (int rc = launch_scan_mode<T, DECAY, SCAN_WHOLE>(p, num_requests, 1, stream)) return rc;
  } else {
    if (int rc = launch_scan_mode<T, DECAY, SCAN_LOCAL>(p, num_requests, p.max_segments, stream)) return rc;
    const int elements = DIM * p.vdim;
    TS_LAUNCH("linear_attention_combine", linear_attention_combine_kernel<DECAY>,
              dim3(num_requests, p.H, (elements + 255) / 256), 256, 0, stream, p);
    if (int rc = launch_scan_mode<T, DECAY, SCAN_FROM_SEGMENT>(p, num_requests, p.max_segments, stream)) return rc;
  }
  if (p.raw_out && p.finish)
    TS_LAUNCH("linear_attention_finish", linear_attention_finish_kernel<T>, num_tokens, p.H >= 8 ? 256 : 128, 0, stream, p,
              num_tokens);
  return 0;
}

}  // namespace

TS_EXPORT int ts_linear_attention_key_dim() { return DIM; }

// value columns of a block: whole warps of column quads (32 / GROUPS quads each), a whole head where it fits
static int block_columns(int vdim) {
  const int step = COLS * (GROUPS >= 32 ? 1 : 32 / GROUPS);
  const int most = MAX_COLS < COLS * MAX_THREADS / GROUPS ? MAX_COLS : COLS * MAX_THREADS / GROUPS;
  const int padded = (vdim + step - 1) / step * step;
  return padded <= most ? padded : most / step * step;
}

// blocks that a head of `vdim` value columns is spread over (more than one: the caller brings a
// 32-bit scratch [T, H * vdim] for the outputs before their norm)
// blocks of the scan that an SM holds at once for heads of `vdim` value columns (128 registers a thread)
TS_EXPORT int ts_linear_attention_resident_blocks(int vdim) {
  const int threads = block_columns(vdim) / COLS * GROUPS;
  const int fit = MAX_THREADS / threads;
  return fit < 1 ? 1 : (fit > 8 ? 8 : fit);
}

TS_EXPORT int ts_linear_attention_column_tiles(int vdim) {
  const int cols = block_columns(vdim);
  return (vdim + cols - 1) / cols;
}

TS_EXPORT int ts_linear_attention(int dtype, const void* q, long long ldq, const void* k, long long ldk, const void* v,
                                  long long ldv, const void* gate, long long ldg, const float* z, long long ldz,
                                  float tau, const float* decay, const int* positions, const float* cos,
                                  const float* sin, int rotary_dim, float q_scale, float k_scale, float* state,
                                  const int* state_slots, const int* fresh, const int* cu_q, int num_requests,
                                  const void* norm_weight, int norm_weight_is_f32, float eps, void* out, long long ldo,
                                  int H, int vdim, int seg_len, float* seg_state, float* seg_decay, int max_segments,
                                  int num_tokens, float* raw_out, int in_act, int gate_act, int joint_norm,
                                  const float* lower, int tied_key, const float* tok_keep, const float* tok_write,
                                  int qk_group, int v_width, int finish, const float* step_raw, long long ld_step,
                                  const void* step_bias, const void* step_rate, int step_vec_is_f32, cudaStream_t stream) {
  TS_REQUIRE(num_requests > 0 && H > 0 && vdim > 0, "linear_attention: empty input");
  TS_REQUIRE(step_raw == nullptr || (step_bias && step_rate && ld_step >= H), "linear_attention: step-size logits come with a bias and a rate per head");
  const int cols = block_columns(vdim);
  const int col_tiles = (vdim + cols - 1) / cols;
  TS_REQUIRE((col_tiles > 1 || joint_norm || !finish) == (raw_out != nullptr) && num_tokens > 0,
             "linear_attention: heads of more than %d value columns, a norm over all heads, and outputs that the caller "
             "finishes, come with a 32-bit scratch for their outputs, others without", cols);
  TS_REQUIRE((z != nullptr) + (decay != nullptr) + (tok_keep != nullptr) + (step_raw != nullptr) == 1,
             "linear_attention: per-channel logits, per-head decays, per-token decays or step-size logits");
  TS_REQUIRE(tok_keep == nullptr || tok_write != nullptr, "linear_attention: per-token decays come with per-token factors on k");
  TS_REQUIRE(z == nullptr || lower != nullptr || tau > 0.f, "linear_attention: tau must be positive");
  TS_REQUIRE(lower == nullptr || z != nullptr, "linear_attention: a lower bound belongs to per-channel logits");
  TS_REQUIRE(!tied_key || (z != nullptr && rotary_dim == 0), "linear_attention: a tied key needs per-channel decays and no rotation");
  TS_REQUIRE(qk_group >= 1 && H % qk_group == 0, "linear_attention: %d heads in groups of %d", H, qk_group);
  TS_REQUIRE(v_width >= 1 && v_width <= vdim && (v_width == vdim || raw_out != nullptr),
             "linear_attention: %d value columns in a state of %d (constant columns: the caller finishes)", v_width, vdim);
  TS_REQUIRE(rotary_dim >= 0 && rotary_dim <= DIM && rotary_dim % 2 == 0, "linear_attention: rotary_dim %d does not fit key size %d", rotary_dim, DIM);
  TS_REQUIRE(rotary_dim == 0 || (cos && sin && positions), "linear_attention: rotary without tables");
  TS_REQUIRE(q && (k || tied_key) && v && (out || !finish) && state && state_slots && fresh && cu_q, "linear_attention: a null operand");
  TS_REQUIRE(seg_len == 0 || (seg_len % CHUNK == 0 && seg_state && max_segments > 0 && max_segments <= 65535 &&
                              (decay != nullptr || seg_decay)),
             "linear_attention: segments of a multiple of %d tokens with scratch for their states", CHUNK);
  ScanParams p{q, k, v, gate, ldq, ldk, ldv, ldg, z, ldz, decay, z && !lower ? 1.f / tau : 0.f, positions, cos, sin, rotary_dim,
               q_scale, k_scale, state, state_slots, fresh, cu_q, norm_weight, norm_weight_is_f32, eps, out, ldo, H, vdim,
               seg_len, seg_state, seg_decay, max_segments, cols, col_tiles, raw_out, in_act, gate_act, joint_norm,
               lower, tied_key, tok_keep, tok_write, qk_group, v_width, finish, step_raw, ld_step,
               VecParam{step_bias, step_vec_is_f32}, VecParam{step_rate, step_vec_is_f32}};
  const int mode = z ? DECAY_CHANNEL : (tok_keep || step_raw ? DECAY_TOKEN : DECAY_HEAD);
  if (dtype == TS_F32) {
    if (mode == DECAY_CHANNEL) return launch_scan<float, DECAY_CHANNEL>(p, num_requests, num_tokens, stream);
    if (mode == DECAY_TOKEN) return launch_scan<float, DECAY_TOKEN>(p, num_requests, num_tokens, stream);
    return launch_scan<float, DECAY_HEAD>(p, num_requests, num_tokens, stream);
  }
  if (dtype == TS_BF16) {
    if (mode == DECAY_CHANNEL) return launch_scan<__nv_bfloat16, DECAY_CHANNEL>(p, num_requests, num_tokens, stream);
    if (mode == DECAY_TOKEN) return launch_scan<__nv_bfloat16, DECAY_TOKEN>(p, num_requests, num_tokens, stream);
    return launch_scan<__nv_bfloat16, DECAY_HEAD>(p, num_requests, num_tokens, stream);
  }
  return ts_fail("linear_attention: unknown dtype %d", dtype);
}
