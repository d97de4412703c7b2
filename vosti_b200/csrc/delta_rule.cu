// Gated delta rule: a recurrent mixer whose state per (request, head) is a float32 matrix
// S [key channels, value channels], with one decay per (head, key channel).
//
// Per token and head, in this order:
//   S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// so the read-out sees the token's own write. Around it: short causal convolutions with SiLU
// on q, k and v (the last taps - 1 inputs of a request are part of its state), q and k made
// unit vectors per head (q also times dk^-1/2), beta = sigmoid(.), g = exp(-exp(A_log) *
// softplus(low-rank(h) + dt_bias)), and an output stage: o divided by its root mean square
// over the value channels, times a weight, times sigmoid(low-rank gate).
//
// Everything after the projections is float32 in both serving types. A request's state slot
// is one float32 vector: S for every head, stored transposed [heads, dv, dk] so that the key
// channels a lane keeps are contiguous, then the convolution tail [taps - 1, conv channels].
//
// Kernels:
//   delta_prep     one warp per (token, q / k / v head): convolutions, unit vectors; beta, decay, gate
//   delta_conv     one block per request: the convolution tail after this step
//   delta_scan     one block per (request, head, block of value columns): the recurrence over
//                  the request's tokens of this step, from and to the state slot. Columns of S
//                  are independent; a column's dk entries are spread over KS lanes of a warp,
//                  R contiguous ones to a lane, and the two sums over them are shuffles.
//   delta_out      one warp per (token, head): the output stage
//
// Two forms of the gated rule share these kernels: the decay is one number per (head, key channel)
// from a low-rank pair, or one number per head from a plain projection (`decay_per_head`: the rates
// then hold `heads` columns, which the preparation spreads over the head's channels); the output
// gate is a sigmoid or SiLU (`gate_silu`); the output weight is shared by the heads or has a row
// per head.
//
// The generalized delta rule (general_prep, general_scan) keeps the same state layout. Per token
// and head, with the unit key u = k / sqrt(|k|^2 + 1e-6), a decay w and a removal rate a per
// (head, key channel):
//   S <- diag(w) S - (a * u) (u^T S) + k v^T     (both first terms read the old S);   o = S^T r
// w = exp(-exp(-1/2) * sigmoid(inner + w0)) with `inner` the product of a low-rank pair with tanh
// between its halves, a = sigmoid(proj_a + bias), gate = sigmoid(proj_g).
#include <stdlib.h>

#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 16;
constexpr int SCAN_THREADS = 256; // most threads of a scan block
constexpr int TOKENS = 16;      // tokens staged in shared memory at a time (in each of two buffers)

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }

struct PrepArgs {
  // the fused projection [tokens, stride]: columns q | k | v | beta
  const void* proj;
  int proj_f32, stride;
  int off_q, off_k, off_v, off_beta;
  // the low-rank pairs' products [tokens, heads dk + heads dv]: decay rates | output gates
  const void* rates;
  int rates_f32;
  int kv_heads, heads, dk, dv, taps;
  const void* conv_w;           // [(2 kv_heads dk + heads dv), taps], the last column is the current token's
  const void* a_log;            // [heads]
  const void* dt_bias;          // [heads dk]
  int w_f32;
  const float* state;           // [slots, state_stride]
  int64_t state_stride, conv_offset;
  const int* request_of;
  const int* cu_q;
  const int* state_slots;
  int num_slots;
  float* q; float* k; float* v; float* beta; float* decay; float* gate;
  unsigned* status;
  int decay_per_head;           // rates: heads decay columns (dt_bias [heads]) instead of heads * dk
  int gate_silu;                // the output gate is z * sigmoid(z) instead of sigmoid(z)
};

// One warp per unit of a token: a q head, a k head or a v head. A lane owns the channels lane,
// lane + 32, ... of its unit, convolves them, and for q and k heads the warp sums the squares
// (a lane's chain, then the fixed tree). blockIdx.y walks the units in groups of the block's
// warps; the element-wise outputs (beta, decay, gate) are spread over the same blocks.
constexpr int PREP_MAX_KEY = 256;            // widest q / k head (8 channels per lane)
__global__ void __launch_bounds__(256) delta_prep_kernel(PrepArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int cq = a.kv_heads * a.dk, cv = a.heads * a.dv, cc = 2 * cq + cv;
  const int b = a.request_of[t];
  const int local = t - a.cu_q[b];
  int slot = a.state_slots[b];
  if (slot < 0 || slot >= a.num_slots) {
    if (threadIdx.x == 0 && blockIdx.y == 0) raise_fault(a.status, VOSTI_FAULT_SLOT_RANGE);
    slot = 0;
  }
  const float* tail = a.state + (int64_t)slot * a.state_stride + a.conv_offset;   // [taps - 1, cc]
  const int64_t row = (int64_t)t * a.stride;
  // q | k | v occupy columns off_q .. off_q + cc of the projection in this order
  auto convolved = [&](int c) {
    float acc = 0.f;
    for (int i = 0; i < a.taps; ++i) {
      const int back = a.taps - 1 - i;                  // how many tokens before this one
      float x;
      if (local - back >= 0) x = load_flex(a.proj, a.proj_f32, row - (int64_t)back * a.stride + a.off_q + c);
      else x = tail[(int64_t)(a.taps - 1 + local - back) * cc + c];
      acc = fmaf(load_flex(a.conv_w, a.w_f32, (int64_t)c * a.taps + i), x, acc);
    }
    return acc * sigmoidf_(acc);
  };
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int units = 2 * a.kv_heads + a.heads;
  for (int unit = blockIdx.y * nwarps + warp; unit < units; unit += gridDim.y * nwarps) {
    if (unit < 2 * a.kv_heads) {
      const int c0 = unit * a.dk;                       // q heads, then k heads
      float y[PREP_MAX_KEY / 32];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < PREP_MAX_KEY / 32; ++j) {
        const int i = lane + 32 * j;
        y[j] = i < a.dk ? convolved(c0 + i) : 0.f;
        ss += y[j] * y[j];
      }
      ss = warp_sum(ss);
      const bool is_q = unit < a.kv_heads;
      const float scale = (1.f / sqrtf(ss + 1e-6f)) * (is_q ? 1.f / sqrtf((float)a.dk) : 1.f);
      float* dst = (is_q ? a.q : a.k) + (int64_t)t * cq + (is_q ? unit : unit - a.kv_heads) * a.dk;
#pragma unroll
      for (int j = 0; j < PREP_MAX_KEY / 32; ++j) {
        const int i = lane + 32 * j;
        if (i < a.dk) dst[i] = y[j] * scale;
      }
    } else {
      const int c0 = (unit - 2 * a.kv_heads) * a.dv;
      for (int i = lane; i < a.dv; i += 32) a.v[(int64_t)t * cv + c0 + i] = convolved(2 * cq + c0 + i);
    }
  }
  const int first = blockIdx.y * blockDim.x + threadIdx.x, step = gridDim.y * blockDim.x;
  for (int h = first; h < a.heads; h += step)
    a.beta[(int64_t)t * a.heads + h] = sigmoidf_(load_flex(a.proj, a.proj_f32, row + a.off_beta + h));
  const int cd = a.heads * a.dk;
  const int rd = a.decay_per_head ? a.heads : cd;           // decay columns of the rates
  const int64_t rrow = (int64_t)t * (rd + cv);
  for (int c = first; c < cd; c += step) {
    const int from = a.decay_per_head ? c / a.dk : c;
    const float rate = load_flex(a.rates, a.rates_f32, rrow + from) + load_flex(a.dt_bias, a.w_f32, from);
    const float speed = expf(load_flex(a.a_log, a.w_f32, c / a.dk));
    a.decay[(int64_t)t * cd + c] = expf(-speed * softplusf_(rate));
  }
  for (int c = first; c < cv; c += step) {
    const float z = load_flex(a.rates, a.rates_f32, rrow + rd + c);
    a.gate[(int64_t)t * cv + c] = a.gate_silu ? z * sigmoidf_(z) : sigmoidf_(z);
  }
}

// The convolution tail of every request after this step: the last taps - 1 rows of
// [old tail ; this step's projection rows]. A thread owns a channel, reads what it needs, then writes.
__global__ void __launch_bounds__(256)
delta_conv_kernel(const void* proj, int proj_f32, int stride, int off_q, int cc, int taps, float* state,
                  int64_t state_stride, int64_t conv_offset, const int* cu_q, const int* state_slots, int num_slots) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const int slot = state_slots[b];
  if (slot < 0 || slot >= num_slots) return;
  const int start = cu_q[b], n = cu_q[b + 1] - start;
  float* tail = state + (int64_t)slot * state_stride + conv_offset;
  const int keep = taps - 1;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < cc; c += gridDim.y * blockDim.x) {
    float next[MAX_TAPS];
    for (int r = 0; r < keep; ++r) {
      const int idx = n + r;                 // row of [old tail (keep rows) ; projection rows (n)]
      next[r] = idx < keep ? tail[(int64_t)idx * cc + c]
                           : load_flex(proj, proj_f32, (int64_t)(start + idx - keep) * stride + off_q + c);
    }
    for (int r = 0; r < keep; ++r) tail[(int64_t)r * cc + c] = next[r];
  }
}

// KS lanes of a warp share a value column; lane part `ks` keeps key channels ks * R .. ks * R + R - 1
// of it. A warp holds 32 / KS columns, a block (its thread count) / KS. Tokens are staged in
// shared memory TOKENS at a time in two buffers: while one block of tokens is computed, the next
// one's k, q, g, v and beta arrive by cp.async. The staged rows of k, q and g are padded with
// zeros to KS * R channels, so a lane reads its R as 16-byte words. Between two tokens the state
// waits for one chain of multiply-adds and one chain of KS-lane shuffles; both wait on the
// shared-memory and shuffle pipe, so R is chosen for few shuffle steps (see the launcher).
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int KS, int R>
__global__ void __launch_bounds__(SCAN_THREADS)
delta_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                  const float* __restrict__ beta, const float* __restrict__ decay, float* __restrict__ out,
                  float* state, int64_t state_stride, const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                  int num_slots, int kv_heads, int heads, int dk, int dv) {
  extern __shared__ __align__(16) float smem[];
  constexpr int PER_WARP = 32 / KS;             // columns of a warp
  constexpr int PAD = KS * R;                   // staged channels per token
  const int threads = blockDim.x;
  const int COLS = threads / KS;                // value columns of a block (8 or more)
  const int STAGE = TOKENS * (3 * PAD + COLS) + TOKENS;      // floats of one buffer (a multiple of 4)
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * COLS;
  const int slot = state_slots[b];
  if (slot < 0 || slot >= num_slots) return;
  const int start = cu_q[b], n = cu_q[b + 1] - start;
  const int g = h / (heads / kv_heads);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ks = lane / PER_WARP, local = warp * PER_WARP + lane % PER_WARP, col = col0 + local;
  const bool live = col < dv;
  const int r0 = ks * R;
  float* S = state + (int64_t)slot * state_stride + ((int64_t)h * dv + col) * dk;     // this column's dk channels
  float s[R];
  const bool wide = (dk % 4 == 0) && live && r0 + R <= dk;
  if (wide) {
#pragma unroll
    for (int i = 0; i < R; i += 4) *reinterpret_cast<float4*>(s + i) = *reinterpret_cast<const float4*>(S + r0 + i);
  } else {
#pragma unroll
    for (int i = 0; i < R; ++i) s[i] = (live && r0 + i < dk) ? S[r0 + i] : 0.f;
  }
  const int cq = kv_heads * dk, cd = heads * dk, cv = heads * dv;
  // 16-byte copies need every row start on a 16-byte boundary
  const bool vec_k = dk % 4 == 0, vec_v = dv % 4 == 0;
  if (PAD != dk) {                                  // the padding stays zero (lanes beyond dk multiply it with zeros)
    for (int i = threadIdx.x; i < 2 * STAGE; i += threads) smem[i] = 0.f;
    __syncthreads();
  }

  auto stage = [&](int t0, int buf) {
    float* sk = smem + buf * STAGE;
    float* sq = sk + TOKENS * PAD;
    float* sg = sq + TOKENS * PAD;
    float* sv = sg + TOKENS * PAD;
    float* sb = sv + TOKENS * COLS;
    const int count = min(TOKENS, n - t0);
    if (vec_k) {
      const int per = dk / 4;
      for (int i = threadIdx.x; i < count * per; i += threads) {
        const int tt = i / per, c = (i % per) * 4;
        const int64_t t = start + t0 + tt;
        cp_async16(sk + tt * PAD + c, k + t * cq + g * dk + c);
        cp_async16(sq + tt * PAD + c, q + t * cq + g * dk + c);
        cp_async16(sg + tt * PAD + c, decay + t * cd + h * dk + c);
      }
    } else {
      for (int i = threadIdx.x; i < count * dk; i += threads) {
        const int tt = i / dk, c = i % dk;
        const int64_t t = start + t0 + tt;
        cp_async4(sk + tt * PAD + c, k + t * cq + g * dk + c);
        cp_async4(sq + tt * PAD + c, q + t * cq + g * dk + c);
        cp_async4(sg + tt * PAD + c, decay + t * cd + h * dk + c);
      }
    }
    if (vec_v) {
      const int per = COLS / 4;
      for (int i = threadIdx.x; i < count * per; i += threads) {
        const int tt = i / per, c = (i % per) * 4;
        if (col0 + c < dv) cp_async16(sv + tt * COLS + c, v + (int64_t)(start + t0 + tt) * cv + h * dv + col0 + c);
      }
    } else {
      for (int i = threadIdx.x; i < count * COLS; i += threads) {
        const int tt = i / COLS, c = i % COLS;
        if (col0 + c < dv) cp_async4(sv + tt * COLS + c, v + (int64_t)(start + t0 + tt) * cv + h * dv + col0 + c);
      }
    }
    for (int i = threadIdx.x; i < count; i += threads) cp_async4(sb + i, beta + (int64_t)(start + t0 + i) * heads + h);
  };

  float* orow = out + (int64_t)start * cv + h * dv + col;
  if (n > 0) stage(0, 0);
  cp_async_commit();
  for (int t0 = 0, buf = 0; t0 < n; t0 += TOKENS, buf ^= 1) {
    if (t0 + TOKENS < n) stage(t0 + TOKENS, buf ^ 1);         // (its last readers passed the barrier below)
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const float* sk = smem + buf * STAGE + r0;
    const float* sq = sk + TOKENS * PAD;
    const float* sg = sq + TOKENS * PAD;
    const float* sv = smem + buf * STAGE + 3 * TOKENS * PAD + local;
    const float* sb = smem + buf * STAGE + 3 * TOKENS * PAD + TOKENS * COLS;
    const int count = min(TOKENS, n - t0);
    for (int tt = 0; tt < count; ++tt) {
      float kt[R], x[R];
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < R; i += 4) {
        *reinterpret_cast<float4*>(kt + i) = *reinterpret_cast<const float4*>(sk + tt * PAD + i);
        *reinterpret_cast<float4*>(x + i) = *reinterpret_cast<const float4*>(sg + tt * PAD + i);
      }
#pragma unroll
      for (int i = 0; i < R; ++i) {
        s[i] *= x[i];
        acc[i & 3] = fmaf(s[i], kt[i], acc[i & 3]);
      }
      float dot = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
      for (int i = 0; i < R; i += 4) *reinterpret_cast<float4*>(x + i) = *reinterpret_cast<const float4*>(sq + tt * PAD + i);
#pragma unroll
      for (int o = PER_WARP; o < 32; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float u = sb[tt] * (sv[tt * COLS] - dot);
      acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        s[i] = fmaf(kt[i], u, s[i]);
        acc[i & 3] = fmaf(s[i], x[i], acc[i & 3]);
      }
      float read = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
      for (int o = PER_WARP; o < 32; o <<= 1) read += __shfl_xor_sync(0xffffffffu, read, o);
      if (ks == 0 && live) orow[(int64_t)(t0 + tt) * cv] = read;
    }
    __syncthreads();                                         // this buffer may be refilled two rounds on
  }
  cp_async_wait<0>();
  if (wide) {
#pragma unroll
    for (int i = 0; i < R; i += 4) *reinterpret_cast<float4*>(S + r0 + i) = *reinterpret_cast<const float4*>(s + i);
  } else {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (live && r0 + i < dk) S[r0 + i] = s[i];
  }
}

// y[t, h, :] = o / sqrt(mean(o^2) + eps) * w * gate, in the serving type, for the output projection.
template <typename TO>
__global__ void __launch_bounds__(128)
delta_out_kernel(const float* __restrict__ o, const float* __restrict__ gate, const void* __restrict__ w, int w_f32,
                 TO* __restrict__ y, int64_t pairs, int dv, float eps, int heads, int w_per_head) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int64_t pair = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (pair >= pairs) return;
  const float* src = o + pair * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss += src[i] * src[i];
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)dv + eps);
  const int64_t wbase = w_per_head ? (pair % heads) * dv : 0;
  for (int i = lane; i < dv; i += 32)
    y[pair * dv + i] = from_f32<TO>(src[i] * inv * load_flex(w, w_f32, wbase + i) * gate[pair * dv + i]);
}


// out[t, j] = tanh(x[t, offset + j]) for j < width: the first half of a low-rank pair whose
// halves have a tanh between them, cut out of a wider projection.
template <typename T>
__global__ void __launch_bounds__(256)
tanh_columns_kernel(const T* __restrict__ x, int stride, int offset, int width, T* __restrict__ out, int64_t tokens) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t n = tokens * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / width;
    out[i] = from_f32<T>(tanhf(to_f32(x[t * stride + offset + (i - t * width)])));
  }
}

struct GeneralPrepArgs {
  const void* proj;             // [tokens, stride]: columns r | k | v | g | a, each heads * d wide
  int proj_f32, stride;
  int off_r, off_k, off_v, off_g, off_a;
  const float* inner;           // [tokens, heads * d]: the decay's low-rank product
  const void* w0;               // [heads * d]
  const void* a_bias;           // [heads * d]
  int w_f32;
  int heads, d;
  float* r; float* k; float* v; float* decay; float* unit; float* removal; float* gate;
};

// One warp per (token, head): blocks of four warps, blockIdx.y over groups of four heads.
__global__ void __launch_bounds__(128) general_prep_kernel(GeneralPrepArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = (int64_t)t * a.stride;
  const int hd = a.heads * a.d;
  const float rate = 0.6065306597126334f;             // exp(-1/2)
  for (int head = blockIdx.y * 4 + warp; head < a.heads; head += gridDim.y * 4) {
    const int c0 = head * a.d;
    float ss = 0.f;
    for (int i = lane; i < a.d; i += 32) {
      const float x = load_flex(a.proj, a.proj_f32, row + a.off_k + c0 + i);
      ss += x * x;
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss + 1e-6f);
    for (int i = lane; i < a.d; i += 32) {
      const int c = c0 + i;
      const int64_t o = (int64_t)t * hd + c;
      const float key = load_flex(a.proj, a.proj_f32, row + a.off_k + c);
      const float u = key * inv;
      a.k[o] = key;
      a.unit[o] = u;
      a.removal[o] = sigmoidf_(load_flex(a.proj, a.proj_f32, row + a.off_a + c) + load_flex(a.a_bias, a.w_f32, c)) * u;
      a.r[o] = load_flex(a.proj, a.proj_f32, row + a.off_r + c);
      a.v[o] = load_flex(a.proj, a.proj_f32, row + a.off_v + c);
      a.decay[o] = expf(-rate * sigmoidf_(a.inner[o] + load_flex(a.w0, a.w_f32, c)));
      a.gate[o] = sigmoidf_(load_flex(a.proj, a.proj_f32, row + a.off_g + c));
    }
  }
}

// The generalized rule's recurrence, laid out as delta_scan: KS lanes share a value column and
// keep R key channels of it each; five vectors of key channels are staged per token (write key,
// read key, decay, unit key, removal = rate * unit key).
template <int KS, int R>
__global__ void __launch_bounds__(SCAN_THREADS)
general_scan_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
                    const float* __restrict__ decay, const float* __restrict__ unit, const float* __restrict__ removal,
                    float* __restrict__ out, float* state, int64_t state_stride, const int* __restrict__ cu_q,
                    const int* __restrict__ state_slots, int num_slots, int heads, int dk, int dv) {
  extern __shared__ __align__(16) float smem[];
  constexpr int PER_WARP = 32 / KS;
  constexpr int PAD = KS * R;
  constexpr int NV = 5;                         // staged vectors of key channels
  const int threads = blockDim.x;
  const int COLS = threads / KS;
  const int STAGE = TOKENS * (NV * PAD + COLS);
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * COLS;
  const int slot = state_slots[b];
  if (slot < 0 || slot >= num_slots) return;
  const int start = cu_q[b], n = cu_q[b + 1] - start;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ks = lane / PER_WARP, local = warp * PER_WARP + lane % PER_WARP, col = col0 + local;
  const bool live = col < dv;
  const int r0 = ks * R;
  float* S = state + (int64_t)slot * state_stride + ((int64_t)h * dv + col) * dk;
  float s[R];
  const bool wide = (dk % 4 == 0) && live && r0 + R <= dk;
  if (wide) {
#pragma unroll
    for (int i = 0; i < R; i += 4) *reinterpret_cast<float4*>(s + i) = *reinterpret_cast<const float4*>(S + r0 + i);
  } else {
#pragma unroll
    for (int i = 0; i < R; ++i) s[i] = (live && r0 + i < dk) ? S[r0 + i] : 0.f;
  }
  const int cd = heads * dk, cv = heads * dv;
  const bool vec_k = dk % 4 == 0, vec_v = dv % 4 == 0;
  if (PAD != dk) {
    for (int i = threadIdx.x; i < 2 * STAGE; i += threads) smem[i] = 0.f;
    __syncthreads();
  }
  const float* sources[NV] = {k, r, decay, unit, removal};

  auto stage = [&](int t0, int buf) {
    float* base = smem + buf * STAGE;
    float* sv = base + NV * TOKENS * PAD;
    const int count = min(TOKENS, n - t0);
    if (vec_k) {
      const int per = dk / 4;
      for (int i = threadIdx.x; i < count * per; i += threads) {
        const int tt = i / per, c = (i % per) * 4;
        const int64_t at = (int64_t)(start + t0 + tt) * cd + h * dk + c;
#pragma unroll
        for (int x = 0; x < NV; ++x) cp_async16(base + x * TOKENS * PAD + tt * PAD + c, sources[x] + at);
      }
    } else {
      for (int i = threadIdx.x; i < count * dk; i += threads) {
        const int tt = i / dk, c = i % dk;
        const int64_t at = (int64_t)(start + t0 + tt) * cd + h * dk + c;
#pragma unroll
        for (int x = 0; x < NV; ++x) cp_async4(base + x * TOKENS * PAD + tt * PAD + c, sources[x] + at);
      }
    }
    if (vec_v) {
      const int per = COLS / 4;
      for (int i = threadIdx.x; i < count * per; i += threads) {
        const int tt = i / per, c = (i % per) * 4;
        if (col0 + c < dv) cp_async16(sv + tt * COLS + c, v + (int64_t)(start + t0 + tt) * cv + h * dv + col0 + c);
      }
    } else {
      for (int i = threadIdx.x; i < count * COLS; i += threads) {
        const int tt = i / COLS, c = i % COLS;
        if (col0 + c < dv) cp_async4(sv + tt * COLS + c, v + (int64_t)(start + t0 + tt) * cv + h * dv + col0 + c);
      }
    }
  };

  float* orow = out + (int64_t)start * cv + h * dv + col;
  if (n > 0) stage(0, 0);
  cp_async_commit();
  for (int t0 = 0, buf = 0; t0 < n; t0 += TOKENS, buf ^= 1) {
    if (t0 + TOKENS < n) stage(t0 + TOKENS, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const float* sk = smem + buf * STAGE + r0;
    const float* sr = sk + TOKENS * PAD;
    const float* sw = sr + TOKENS * PAD;
    const float* su = sw + TOKENS * PAD;
    const float* sa = su + TOKENS * PAD;
    const float* sv = smem + buf * STAGE + NV * TOKENS * PAD + local;
    const int count = min(TOKENS, n - t0);
    for (int tt = 0; tt < count; ++tt) {
      float x[R], y[R];
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < R; i += 4) *reinterpret_cast<float4*>(x + i) = *reinterpret_cast<const float4*>(su + tt * PAD + i);
#pragma unroll
      for (int i = 0; i < R; ++i) acc[i & 3] = fmaf(s[i], x[i], acc[i & 3]);
      float dot = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
      for (int i = 0; i < R; i += 4) {
        *reinterpret_cast<float4*>(x + i) = *reinterpret_cast<const float4*>(sw + tt * PAD + i);
        *reinterpret_cast<float4*>(y + i) = *reinterpret_cast<const float4*>(sa + tt * PAD + i);
      }
#pragma unroll
      for (int o = PER_WARP; o < 32; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float value = sv[tt * COLS];
#pragma unroll
      for (int i = 0; i < R; ++i) s[i] = fmaf(-y[i], dot, s[i] * x[i]);
#pragma unroll
      for (int i = 0; i < R; i += 4) {
        *reinterpret_cast<float4*>(x + i) = *reinterpret_cast<const float4*>(sk + tt * PAD + i);
        *reinterpret_cast<float4*>(y + i) = *reinterpret_cast<const float4*>(sr + tt * PAD + i);
      }
      acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        s[i] = fmaf(x[i], value, s[i]);
        acc[i & 3] = fmaf(s[i], y[i], acc[i & 3]);
      }
      float read = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
      for (int o = PER_WARP; o < 32; o <<= 1) read += __shfl_xor_sync(0xffffffffu, read, o);
      if (ks == 0 && live) orow[(int64_t)(t0 + tt) * cv] = read;
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  if (wide) {
#pragma unroll
    for (int i = 0; i < R; i += 4) *reinterpret_cast<float4*>(S + r0 + i) = *reinterpret_cast<const float4*>(s + i);
  } else {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (live && r0 + i < dk) S[r0 + i] = s[i];
  }
}

}  // namespace

VOSTI_API int vosti_delta_prep(const void* proj, int proj_f32, int stride, int off_q, int off_k, int off_v, int off_beta,
                               const void* rates, int rates_f32, int kv_heads, int heads, int dk, int dv, int taps,
                               const void* conv_w, const void* a_log, const void* dt_bias, int w_f32, float* state,
                               int64_t state_stride, int64_t conv_offset, const int* request_of, const int* cu_q,
                               const int* state_slots, int num_slots, int requests, int tokens, float* q, float* k,
                               float* v, float* beta, float* decay, float* gate, unsigned* status, int decay_per_head,
                               int gate_silu, cudaStream_t stream) {
  VOSTI_REQUIRE(kv_heads > 0 && heads > 0 && heads % kv_heads == 0 && dk > 0 && dv > 0, "delta_prep: bad head sizes");
  VOSTI_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "delta_prep: %d taps (1 to %d are taken)", taps, MAX_TAPS);
  VOSTI_REQUIRE(off_k == off_q + kv_heads * dk && off_v == off_k + kv_heads * dk, "delta_prep: q, k, v must be adjacent columns");
  if (tokens == 0) return VOSTI_OK;
  PrepArgs a = {};
  a.proj = proj; a.proj_f32 = proj_f32; a.stride = stride;
  a.off_q = off_q; a.off_k = off_k; a.off_v = off_v; a.off_beta = off_beta;
  a.rates = rates; a.rates_f32 = rates_f32;
  a.kv_heads = kv_heads; a.heads = heads; a.dk = dk; a.dv = dv; a.taps = taps;
  a.conv_w = conv_w; a.a_log = a_log; a.dt_bias = dt_bias; a.w_f32 = w_f32;
  a.state = state; a.state_stride = state_stride; a.conv_offset = conv_offset;
  a.request_of = request_of; a.cu_q = cu_q; a.state_slots = state_slots; a.num_slots = num_slots;
  a.q = q; a.k = k; a.v = v; a.beta = beta; a.decay = decay; a.gate = gate; a.status = status;
  a.decay_per_head = decay_per_head; a.gate_silu = gate_silu;
  const int cc = 2 * kv_heads * dk + heads * dv;
  VOSTI_REQUIRE(dk <= PREP_MAX_KEY, "delta_prep: %d key channels (at most %d are taken)", dk, PREP_MAX_KEY);
  const int units = 2 * kv_heads + heads;
  vosti_launch(delta_prep_kernel, dim3(tokens, (units + 7) / 8 < 65535 ? (units + 7) / 8 : 65535), dim3(256), 0, stream, a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { vosti_set_error("%s", cudaGetErrorString(e)); return (int)e; }
  // the tail is rewritten only after every token of the step has read the old one
  if (taps > 1)
    vosti_launch(delta_conv_kernel, dim3(requests, (cc + 255) / 256 < 64 ? (cc + 255) / 256 : 64), dim3(256), 0, stream, proj, proj_f32, stride, off_q, cc, taps, state,
                 state_stride, conv_offset, cu_q, state_slots, num_slots);
  VOSTI_LAUNCH_CHECK();
}

// How many key channels a lane keeps (8, 16 or 32). VOSTI_SCAN_ROWS overrides the rule (tuning).
static int scan_rows(int dk) {
  static int forced = -1;
  if (forced < 0) {
    const char* env = getenv("VOSTI_SCAN_ROWS");
    forced = env != nullptr ? atoi(env) : 0;
  }
  if ((forced == 8 || forced == 16 || forced == 32) && dk <= forced * 32 && (forced != 32 || dk <= 256)) return forced;
  return dk <= 32 ? 8 : 16;
}

VOSTI_API int vosti_delta_scan(const float* q, const float* k, const float* v, const float* beta, const float* decay,
                               float* out, float* state, int64_t state_stride, const int* cu_q, const int* state_slots,
                               int num_slots, int requests, int kv_heads, int heads, int dk, int dv, cudaStream_t stream) {
  VOSTI_REQUIRE(kv_heads > 0 && heads > 0 && heads % kv_heads == 0 && dk > 0 && dv > 0, "delta_scan: bad head sizes");
  VOSTI_REQUIRE(dk <= 256, "delta_scan: %d key channels (at most 256 are taken)", dk);
  VOSTI_REQUIRE(heads <= 65535, "delta_scan: too many heads");
  VOSTI_REQUIRE(state_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(state) & 15) == 0, "delta_scan: state slots must be 16-byte aligned");
  if (requests == 0) return VOSTI_OK;
  const int rows = scan_rows(dk);
  int ks = 1;
  while (ks * rows < dk) ks *= 2;
  // blocks of 8 columns or more; smaller blocks while the grid would leave SMs idle
  int threads = SCAN_THREADS;
  while (threads > 64 && threads / 2 >= 8 * ks &&
         (int64_t)requests * heads * ((dv + threads / ks - 1) / (threads / ks)) < 296)
    threads /= 2;
  if (threads < 8 * ks) threads = 8 * ks;
  const int cols = threads / ks;
  VOSTI_REQUIRE((dv + cols - 1) / cols <= 65535, "delta_scan: too many value channels");
  const dim3 grid(requests, heads, (dv + cols - 1) / cols);
  const size_t smem = 2 * (size_t)(TOKENS * (3 * ks * rows + cols) + TOKENS) * sizeof(float);
#define VOSTI_SCAN(KS, R)                                                                                           \
  do {                                                                                                              \
    static bool configured = false;    /* once per instantiation, to the most a launch of it may ask for */           \
    if (!configured) {                                                                                              \
      cudaFuncSetAttribute(delta_scan_kernel<KS, R>, cudaFuncAttributeMaxDynamicSharedMemorySize,                   \
                           (int)(2 * (size_t)(TOKENS * (3 * KS * R + SCAN_THREADS / KS) + TOKENS) * sizeof(float))); \
      configured = true;                                                                                            \
    }                                                                                                               \
    vosti_launch(delta_scan_kernel<KS, R>, grid, dim3(threads), smem, stream, q, k, v, beta, decay, out, state,    \
                 state_stride, cu_q, state_slots, num_slots, kv_heads, heads, dk, dv);                              \
  } while (0)
#define VOSTI_SCAN_KS(R)                                                                                            \
  switch (ks) {                                                                                                     \
    case 1: VOSTI_SCAN(1, R); break;                                                                                \
    case 2: VOSTI_SCAN(2, R); break;                                                                                \
    case 4: VOSTI_SCAN(4, R); break;                                                                                \
    case 8: VOSTI_SCAN(8, R); break;                                                                                \
    case 16: VOSTI_SCAN(16, R); break;                                                                              \
    default: VOSTI_SCAN(32, R); break;                                                                              \
  }
  if (rows == 8) { VOSTI_SCAN_KS(8) } else if (rows == 16) { VOSTI_SCAN_KS(16) } else { VOSTI_SCAN_KS(32) }
#undef VOSTI_SCAN_KS
#undef VOSTI_SCAN
  VOSTI_LAUNCH_CHECK();
}

VOSTI_API int vosti_delta_out(const float* o, const float* gate, const void* w, int w_f32, void* y, int y_f32, int tokens,
                              int heads, int dv, float eps, int w_per_head, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && heads > 0 && dv > 0, "delta_out: bad sizes");
  if (tokens == 0) return VOSTI_OK;
  const int64_t pairs = (int64_t)tokens * heads;
  const unsigned blocks = (unsigned)((pairs + 3) / 4);
  if (y_f32) vosti_launch(delta_out_kernel<float>, dim3(blocks), dim3(128), 0, stream, o, gate, w, w_f32, (float*)y, pairs, dv, eps, heads, w_per_head);
  else vosti_launch(delta_out_kernel<bf16>, dim3(blocks), dim3(128), 0, stream, o, gate, w, w_f32, (bf16*)y, pairs, dv, eps, heads, w_per_head);
  VOSTI_LAUNCH_CHECK();
}

// proj [tokens, stride] (serving type) holds r | k | v | g | a at the given offsets; inner float32
// [tokens, heads * d]; outputs float32 [tokens, heads * d] each.
VOSTI_API int vosti_general_delta_prep(const void* proj, int proj_f32, int stride, int off_r, int off_k, int off_v, int off_g,
                                       int off_a, const float* inner, const void* w0, const void* a_bias, int w_f32,
                                       int heads, int d, int tokens, float* r, float* k, float* v, float* decay, float* unit,
                                       float* removal, float* gate, cudaStream_t stream) {
  VOSTI_REQUIRE(heads > 0 && d > 0 && tokens >= 0, "general_delta_prep: bad sizes");
  if (tokens == 0) return VOSTI_OK;
  GeneralPrepArgs a = {};
  a.proj = proj; a.proj_f32 = proj_f32; a.stride = stride;
  a.off_r = off_r; a.off_k = off_k; a.off_v = off_v; a.off_g = off_g; a.off_a = off_a;
  a.inner = inner; a.w0 = w0; a.a_bias = a_bias; a.w_f32 = w_f32; a.heads = heads; a.d = d;
  a.r = r; a.k = k; a.v = v; a.decay = decay; a.unit = unit; a.removal = removal; a.gate = gate;
  VOSTI_REQUIRE((heads + 3) / 4 <= 65535, "general_delta_prep: too many heads");
  vosti_launch(general_prep_kernel, dim3(tokens, (heads + 3) / 4), dim3(128), 0, stream, a);
  VOSTI_LAUNCH_CHECK();
}

VOSTI_API int vosti_general_delta_scan(const float* r, const float* k, const float* v, const float* decay, const float* unit,
                                       const float* removal, float* out, float* state, int64_t state_stride, const int* cu_q,
                                       const int* state_slots, int num_slots, int requests, int heads, int dk, int dv,
                                       cudaStream_t stream) {
  VOSTI_REQUIRE(heads > 0 && dk > 0 && dv > 0, "general_delta_scan: bad head sizes");
  VOSTI_REQUIRE(dk <= 256, "general_delta_scan: %d key channels (at most 256 are taken)", dk);
  VOSTI_REQUIRE(heads <= 65535, "general_delta_scan: too many heads");
  VOSTI_REQUIRE(state_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(state) & 15) == 0, "general_delta_scan: state slots must be 16-byte aligned");
  if (requests == 0) return VOSTI_OK;
  const int rows = scan_rows(dk);
  int ks = 1;
  while (ks * rows < dk) ks *= 2;
  int threads = SCAN_THREADS;
  while (threads > 64 && threads / 2 >= 8 * ks &&
         (int64_t)requests * heads * ((dv + threads / ks - 1) / (threads / ks)) < 296)
    threads /= 2;
  if (threads < 8 * ks) threads = 8 * ks;
  const int cols = threads / ks;
  VOSTI_REQUIRE((dv + cols - 1) / cols <= 65535, "general_delta_scan: too many value channels");
  const dim3 grid(requests, heads, (dv + cols - 1) / cols);
  const size_t smem = 2 * (size_t)(TOKENS * (5 * ks * rows + cols)) * sizeof(float);
#define VOSTI_SCAN(KS, R)                                                                                           \
  do {                                                                                                              \
    static bool configured = false;                                                                                 \
    if (!configured) {                                                                                              \
      cudaFuncSetAttribute(general_scan_kernel<KS, R>, cudaFuncAttributeMaxDynamicSharedMemorySize,                 \
                           (int)(2 * (size_t)(TOKENS * (5 * KS * R + SCAN_THREADS / KS)) * sizeof(float)));          \
      configured = true;                                                                                            \
    }                                                                                                               \
    vosti_launch(general_scan_kernel<KS, R>, grid, dim3(threads), smem, stream, r, k, v, decay, unit, removal, out, \
                 state, state_stride, cu_q, state_slots, num_slots, heads, dk, dv);                                 \
  } while (0)
#define VOSTI_SCAN_KS(R)                                                                                            \
  switch (ks) {                                                                                                     \
    case 1: VOSTI_SCAN(1, R); break;                                                                                \
    case 2: VOSTI_SCAN(2, R); break;                                                                                \
    case 4: VOSTI_SCAN(4, R); break;                                                                                \
    case 8: VOSTI_SCAN(8, R); break;                                                                                \
    case 16: VOSTI_SCAN(16, R); break;                                                                              \
    default: VOSTI_SCAN(32, R); break;                                                                              \
  }
  if (rows == 8) { VOSTI_SCAN_KS(8) } else if (rows == 16) { VOSTI_SCAN_KS(16) } else { VOSTI_SCAN_KS(32) }
#undef VOSTI_SCAN_KS
#undef VOSTI_SCAN
  VOSTI_LAUNCH_CHECK();
}

VOSTI_API int vosti_tanh_columns(const void* x, int is_f32, int stride, int offset, int width, void* out, int tokens,
                                 cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && width > 0 && offset >= 0 && offset + width <= stride, "tanh_columns: bad sizes");
  if (tokens == 0) return VOSTI_OK;
  const int64_t n = (int64_t)tokens * width;
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  if (is_f32) vosti_launch(tanh_columns_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, stride, offset, width, (float*)out, (int64_t)tokens);
  else vosti_launch(tanh_columns_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)x, stride, offset, width, (bf16*)out, (int64_t)tokens);
  VOSTI_LAUNCH_CHECK();
}
