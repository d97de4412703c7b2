// Mixture of experts: the router's choice and what it costs to apply it.
//
// moe_route: per token, the `top` experts with the largest float32 router logits (the lowest
// index wins a tie) and their weights, the softmax over the chosen logits only. It writes the
// choice twice: as lists (expert ids and weights, [tokens, top]) and as a dense float32 matrix
// [tokens, experts] that is zero where an expert was not chosen.
//
// moe_scale: multiplies each expert's slice of the stacked activation [tokens, experts * ff] by
// the token's weight for that expert (zero for experts it did not choose), so that one product
// with the experts' down projections side by side, [width, experts * ff], is the weighted sum
// of the chosen experts' outputs.
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int tokens, int experts, int top, int* __restrict__ chosen,
                 float* __restrict__ weights, float* __restrict__ dense) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const float* row = logits + (int64_t)t * experts;
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
  const float inv = 1.f / total;
  if (lane == 0)
    for (int r = 0; r < top; ++r) {
      const float w = weights[(int64_t)t * top + r] * inv;
      weights[(int64_t)t * top + r] = w;
      dense[(int64_t)t * experts + chosen[(int64_t)t * top + r]] = w;
    }
}

template <typename T>
__global__ void moe_scale_kernel(T* __restrict__ act, const float* __restrict__ dense, int64_t tokens, int experts, int ff) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t width = (int64_t)experts * ff, n = tokens * width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / width;
    const int e = (int)((i - t * width) / ff);
    act[i] = from_f32<T>(to_f32(act[i]) * dense[t * experts + e]);
  }
}

}  // namespace

VOSTI_API int vosti_moe_route(const float* logits, int tokens, int experts, int top, int* chosen, float* weights,
                              float* dense, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && experts > 0 && top > 0 && top <= experts, "moe_route: bad sizes experts=%d top=%d", experts, top);
  VOSTI_REQUIRE(experts <= 2048, "moe_route: %d experts (at most 2048 are taken)", experts);
  if (tokens == 0) return VOSTI_OK;
  vosti_launch(moe_route_kernel, dim3((tokens + 3) / 4), dim3(128), 0, stream, logits, tokens, experts, top, chosen, weights, dense);
  VOSTI_LAUNCH_CHECK();
}

VOSTI_API int vosti_moe_scale(void* act, const float* dense, int tokens, int experts, int ff, int is_f32, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && experts > 0 && ff > 0, "moe_scale: bad sizes");
  if (tokens == 0) return VOSTI_OK;
  const int64_t n = (int64_t)tokens * experts * ff;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  if (is_f32) vosti_launch(moe_scale_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)act, dense, (int64_t)tokens, experts, ff);
  else vosti_launch(moe_scale_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (bf16*)act, dense, (int64_t)tokens, experts, ff);
  VOSTI_LAUNCH_CHECK();
}
