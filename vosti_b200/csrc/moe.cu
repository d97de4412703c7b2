// Mixture of experts: the router's choice and what it costs to apply it.
//
// moe_route: per token, the `top` experts with the largest float32 router logits (the lowest
// index wins a tie) and their weights: the softmax over the chosen logits only, or (`over_all`)
// the softmax over all experts, of which the chosen ones' scores are divided by their sum (plus
// 1e-20); either way times a constant `scale`. It writes the
// choice twice: as lists (expert ids and weights, [tokens, top]) and as a dense float32 matrix
// [tokens, experts] that is zero where an expert was not chosen.
//
// moe_scale: multiplies each expert's slice of the stacked activation [tokens, experts * ff] by
// the token's weight for that expert (zero for experts it did not choose), after an optional
// activation of its own (the exact GELU, for experts without a gate), so that one product
// with the experts' down projections side by side, [width, experts * ff], is the weighted sum
// of the chosen experts' outputs.
//
// For long portions the stacked product would compute every expert for every token. There the
// (token, pick) pairs are sorted by expert instead (moe_group: one block counts, scans and
// places them, so the order inside an expert's run is by pair index and the same every time),
// every expert multiplies its own run of gathered rows, and moe_combine adds a token's picks in
// the order of its picks: out[t] = sum_k w[t, k] * y[where[t, k]].
#include "common.cuh"

namespace {

// One warp: the choice for token t from its row of logits (global or shared memory).
__device__ __forceinline__ void route_row(const float* row, int t, int experts, int top, int* __restrict__ chosen,
                                          float* __restrict__ weights, float* __restrict__ dense, int over_all, float scale) {
  const int lane = threadIdx.x & 31;
  for (int e = lane; e < experts; e += 32) dense[(int64_t)t * experts + e] = 0.f;
  float first = 0.f, total = 0.f;
  unsigned long long taken_low = 0;     // experts 0..63 this lane already gave away (bit e / 32 of its share)
  for (int r = 0; r < top; ++r) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane, n = 0; e < experts; e += 32, ++n) {
      const bool taken = n < 64 ? (taken_low >> n) & 1ull : false;
      const float v = row[e];
      if (!taken && (v > best || (v == best && e < best_e))) { best = v; best_e = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
    }
    if (best_e != 0x7fffffff && (best_e & 31) == lane) taken_low |= 1ull << (best_e >> 5);
    if (r == 0) first = best;
    const float p = expf(best - first);        // the first pick is the largest logit
    total += p;
    if (lane == 0) {
      chosen[(int64_t)t * top + r] = best_e;
      weights[(int64_t)t * top + r] = p;
    }
  }
  __syncwarp();
  float inv = 1.f / total;
  if (over_all) {
    // scores over all experts: exp(z - max) / Z; the chosen ones' sum is total / Z
    float z = 0.f;
    for (int e = lane; e < experts; e += 32) z += expf(row[e] - first);
    z = warp_sum(z);
    inv = (1.f / z) / (total / z + 1e-20f);
  }
  inv *= scale;
  if (lane == 0)
    for (int r = 0; r < top; ++r) {
      const float w = weights[(int64_t)t * top + r] * inv;
      weights[(int64_t)t * top + r] = w;
      dense[(int64_t)t * experts + chosen[(int64_t)t * top + r]] = w;
    }
}

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int tokens, int experts, int top, int* __restrict__ chosen,
                 float* __restrict__ weights, float* __restrict__ dense, int over_all, float scale) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= tokens) return;
  route_row(logits + (int64_t)t * experts, t, experts, top, chosen, weights, dense, over_all, scale);
}

// The router's product and the choice in one kernel, one block per token: the token's row goes to
// shared memory as float32, every warp makes the logits of its experts (a lane's multiply-add
// chain over k = lane, lane + 32, ..., then the warp's fixed tree: the order depends on k alone),
// and the first warp chooses. The router's matrix is float32 [experts, k].
__global__ void __launch_bounds__(256)
moe_router_kernel(const void* __restrict__ x, int x_f32, const float* __restrict__ router, int experts, int k, int top,
                  int* __restrict__ chosen, float* __restrict__ weights, float* __restrict__ dense, float* __restrict__ logits,
                  int over_all, float scale) {
  extern __shared__ __align__(16) float router_smem[];         // [k] the token's row, then [experts] its logits
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* xs = router_smem;
  float* lg = router_smem + k;
  for (int i = threadIdx.x; i < k; i += blockDim.x) xs[i] = load_flex(x, x_f32, (int64_t)t * k + i);
  __syncthreads();
  const int nwarps = blockDim.x >> 5;
  for (int e = warp; e < experts; e += nwarps) {
    const float* w = router + (int64_t)e * k;
    float acc = 0.f;
    if (k % 4 == 0) {
      // 16-byte words, four of them in flight: a lane's chain runs over the words lane, lane + 32, ...
      float part[4] = {0.f, 0.f, 0.f, 0.f};
      const float4* w4 = reinterpret_cast<const float4*>(w);
      const float4* x4 = reinterpret_cast<const float4*>(xs);
#pragma unroll 4
      for (int i = lane; i < k / 4; i += 32) {
        const float4 a = x4[i], b = w4[i];
        part[0] = fmaf(a.x, b.x, part[0]);
        part[1] = fmaf(a.y, b.y, part[1]);
        part[2] = fmaf(a.z, b.z, part[2]);
        part[3] = fmaf(a.w, b.w, part[3]);
      }
      acc = (part[0] + part[1]) + (part[2] + part[3]);
    } else {
      for (int i = lane; i < k; i += 32) acc = fmaf(xs[i], w[i], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      lg[e] = acc;
      if (logits != nullptr) logits[(int64_t)t * experts + e] = acc;
    }
  }
  __syncthreads();
  if (warp == 0) route_row(lg, t, experts, top, chosen, weights, dense, over_all, scale);
}

// `dense` null: the activation alone.
template <typename T>
__global__ void moe_scale_kernel(T* __restrict__ act, const float* __restrict__ dense, int64_t tokens, int experts, int ff,
                                 int gelu) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t width = (int64_t)experts * ff, n = tokens * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / width;
    const int e = (int)((i - t * width) / ff);
    float x = to_f32(act[i]);
    if (gelu) x = 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
    if (dense != nullptr) x *= dense[t * experts + e];
    act[i] = from_f32<T>(x);
  }
}

// One block. chosen: [pairs] expert of every (token, pick) pair, pair = token * top + pick.
// offsets [experts + 1]: where each expert's run starts in the sorted order; rows [pairs]: the
// token of the pair at each sorted place; where [pairs]: the sorted place of each pair.
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ chosen, int pairs, int top, int experts, int* __restrict__ offsets,
                 int* __restrict__ rows, int* __restrict__ where) {
  extern __shared__ int counts[];           // [experts + 1]
  pdl_wait();
  pdl_launch_dependents();
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = chosen[i];
    if (e >= 0 && e < experts) atomicAdd(&counts[e + 1], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int e = 0; e < experts; ++e) counts[e + 1] += counts[e];
    for (int e = 0; e <= experts; ++e) offsets[e] = counts[e];
  }
  __syncthreads();
  // a pair's place: its expert's start plus the number of earlier pairs of the same expert.
  // One warp per expert walks the pairs in order, so the placement never varies.
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int e = warp; e < experts; e += nwarps) {
    int at = counts[e];
    for (int i0 = 0; i0 < pairs; i0 += 32) {
      const int i = i0 + lane;
      const bool mine = i < pairs && chosen[i] == e;
      const unsigned ballot = __ballot_sync(0xffffffffu, mine);
      if (mine) {
        const int place = at + __popc(ballot & ((1u << lane) - 1u));
        rows[place] = i / top;
        where[i] = place;
      }
      at += __popc(ballot);
    }
  }
}

__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ where, const float* __restrict__ weights,
                   float* __restrict__ out, int top, int width) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k)
      acc = fmaf(weights[(int64_t)t * top + k], y[(int64_t)where[(int64_t)t * top + k] * width + c], acc);
    out[(int64_t)t * width + c] = acc;
  }
}

}  // namespace

VOSTI_API int vosti_moe_group(const int* chosen, int tokens, int top, int experts, int* offsets, int* rows, int* where,
                              cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && top > 0 && experts > 0 && experts <= 8192, "moe_group: bad sizes");
  VOSTI_REQUIRE((int64_t)tokens * top < (int64_t)1 << 30, "moe_group: too many pairs");
  vosti_launch(moe_group_kernel, dim3(1), dim3(1024), (size_t)(experts + 1) * sizeof(int), stream, chosen, tokens * top, top,
               experts, offsets, rows, where);
  VOSTI_LAUNCH_CHECK();
}

VOSTI_API int vosti_moe_combine(const float* y, const int* where, const float* weights, float* out, int tokens, int top,
                                int width, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && top > 0 && width > 0, "moe_combine: bad sizes");
  if (tokens == 0) return VOSTI_OK;
  vosti_launch(moe_combine_kernel, dim3(tokens), dim3(256), 0, stream, y, where, weights, out, top, width);
  VOSTI_LAUNCH_CHECK();
}

VOSTI_API int vosti_moe_route(const float* logits, int tokens, int experts, int top, int* chosen, float* weights,
                              float* dense, int over_all, float scale, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && experts > 0 && top > 0 && top <= experts, "moe_route: bad sizes experts=%d top=%d", experts, top);
  VOSTI_REQUIRE(experts <= 2048, "moe_route: %d experts (at most 2048 are taken)", experts);
  if (tokens == 0) return VOSTI_OK;
  vosti_launch(moe_route_kernel, dim3((tokens + 3) / 4), dim3(128), 0, stream, logits, tokens, experts, top, chosen, weights, dense, over_all, scale);
  VOSTI_LAUNCH_CHECK();
}

VOSTI_API int vosti_moe_scale(void* act, const float* dense, int tokens, int experts, int ff, int is_f32, int gelu,
                              cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && experts > 0 && ff > 0, "moe_scale: bad sizes");
  if (tokens == 0) return VOSTI_OK;
  const int64_t n = (int64_t)tokens * experts * ff;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  if (is_f32) vosti_launch(moe_scale_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)act, dense, (int64_t)tokens, experts, ff, gelu);
  else vosti_launch(moe_scale_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (bf16*)act, dense, (int64_t)tokens, experts, ff, gelu);
  VOSTI_LAUNCH_CHECK();
}

// x [tokens, k] float32 or bfloat16; router float32 [experts, k]; `logits` (optional) receives the
// float32 logits [tokens, experts].
VOSTI_API int vosti_moe_router(const void* x, int x_f32, const float* router, int tokens, int experts, int k, int top,
                               int* chosen, float* weights, float* dense, float* logits, int over_all, float scale,
                               cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && experts > 0 && top > 0 && top <= experts && k > 0, "moe_router: bad sizes experts=%d top=%d", experts, top);
  VOSTI_REQUIRE(experts <= 2048, "moe_router: %d experts (at most 2048 are taken)", experts);
  const size_t smem = (size_t)(k + experts) * sizeof(float);
  VOSTI_REQUIRE(smem <= 200 * 1024, "moe_router: a row of %d elements does not fit shared memory", k);
  if (tokens == 0) return VOSTI_OK;
  {
    static bool configured = false;       // once, to the most a launch may ask for
    if (!configured) {
      cudaFuncSetAttribute(moe_router_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      configured = true;
    }
  }
  vosti_launch(moe_router_kernel, dim3(tokens), dim3(experts > 4 ? 256 : 128), smem, stream, x, x_f32, router, experts, k, top, chosen, weights,
               dense, logits, over_all, scale);
  VOSTI_LAUNCH_CHECK();
}
