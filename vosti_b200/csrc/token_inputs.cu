// What a model takes from the token ids themselves besides the embedding row:
//
// pair_embedding: x[t] = table[id] + pairs[row] in float32, where row hashes the token with the
// one before it in its sequence, (prev * mul_prev + id * mul_cur) mod buckets, and a sequence's
// first token (position 0) takes the row after the hashed ones (row `buckets`). The token before
// the first one of a step's portion is the last token of the request's step before: it lives in
// the request's state slot (one int32), which pair_state rewrites after every token of the step
// has been read. Token ids a sampler left on the device (`source`, `values`: see the embedding
// kernel) are resolved here, and the resolved ids are stored for the layers that read them again.
//
// token_gate: g[t, j] = gelu_tanh(z[t, j]) * side[id_t, offset + j], the gate of a per-layer
// token input: every layer owns `dim` columns of a table of per-token vectors.
#include "common.cuh"

namespace {

__device__ __forceinline__ int resolve_id(const int* ids, const int* source, const int* values, int t) {
  return (source != nullptr && source[t] >= 0) ? values[source[t]] : ids[t];
}

template <typename T>
__global__ void __launch_bounds__(128)
pair_embedding_kernel(const int* __restrict__ ids, const int* __restrict__ source, const int* __restrict__ values,
                      const int* __restrict__ positions, const int* __restrict__ request_of, const int* __restrict__ cu_q,
                      const int* __restrict__ state_slots, const int* __restrict__ last_token, int num_slots,
                      const T* __restrict__ table, const T* __restrict__ pairs, float* __restrict__ out,
                      int* __restrict__ resolved, int hidden, int vocab, long long buckets, long long mul_prev,
                      long long mul_cur, unsigned* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = resolve_id(ids, source, values, t);
  bool bad = id < 0 || id >= vocab;
  if (bad) id = 0;
  long long row = buckets;
  if (positions[t] > 0) {
    const int b = request_of[t];
    int prev;
    if (t == cu_q[b]) {
      const int slot = state_slots[b];
      if (slot < 0 || slot >= num_slots) {
        if (threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_SLOT_RANGE);
        prev = 0;
      } else {
        prev = last_token[slot];
      }
    } else {
      prev = resolve_id(ids, source, values, t - 1);
    }
    if (prev < 0 || prev >= vocab) { bad = true; prev = 0; }
    row = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
  }
  if (bad && threadIdx.x == 0) raise_fault(status, VOSTI_FAULT_TOKEN_RANGE);
  if (threadIdx.x == 0) resolved[t] = id;
  const T* a = table + (int64_t)id * hidden;
  const T* p = pairs + row * hidden;
  float* dst = out + (int64_t)t * hidden;
  if (sizeof(T) == 2 && hidden % 8 == 0 && !bad) {          // 16-byte words of bfloat16
    const uint4* a8 = reinterpret_cast<const uint4*>(a);
    const uint4* p8 = reinterpret_cast<const uint4*>(p);
    for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
      const uint4 ra = a8[i], rp = p8[i];
      const __nv_bfloat162* xa = reinterpret_cast<const __nv_bfloat162*>(&ra);
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&rp);
      float r[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 fa = __bfloat1622float2(xa[e]), fp = __bfloat1622float2(xp[e]);
        r[2 * e] = fa.x + fp.x;
        r[2 * e + 1] = fa.y + fp.y;
      }
      reinterpret_cast<float4*>(dst)[2 * i] = make_float4(r[0], r[1], r[2], r[3]);
      reinterpret_cast<float4*>(dst)[2 * i + 1] = make_float4(r[4], r[5], r[6], r[7]);
    }
    return;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = bad ? 0.f : to_f32(a[i]) + to_f32(p[i]);
}

// One thread per request: the last token of its portion becomes the slot's last token.
__global__ void pair_state_kernel(const int* __restrict__ resolved, const int* __restrict__ cu_q,
                                  const int* __restrict__ state_slots, int* __restrict__ last_token, int num_slots,
                                  int requests) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= requests) return;
  const int slot = state_slots[b];
  const int end = cu_q[b + 1];
  if (slot < 0 || slot >= num_slots || end <= cu_q[b]) return;
  last_token[slot] = resolved[end - 1];
}

__device__ __forceinline__ float gelu_tanh_(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T, typename TS>
__global__ void __launch_bounds__(256)
token_gate_kernel(const T* __restrict__ z, const int* __restrict__ ids, const TS* __restrict__ side, int64_t side_stride,
                  int offset, int dim, int vocab, T* __restrict__ out, int64_t tokens) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t n = tokens * dim;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / dim;
    const int j = (int)(i - t * dim);
    int id = ids[t];
    if (id < 0 || id >= vocab) id = 0;          // (the embedding has reported it)
    out[i] = from_f32<T>(gelu_tanh_(to_f32(z[i])) * to_f32(side[(int64_t)id * side_stride + offset + j]));
  }
}

}  // namespace

// table [vocab, hidden] and pairs [buckets + 1, hidden] share a type; out float32 [tokens, hidden];
// resolved int32 [tokens]; last_token int32 [num_slots] (a view with stride 1).
VOSTI_API int vosti_pair_embedding(const int* ids, const int* source, const int* values, const int* positions,
                                   const int* request_of, const int* cu_q, const int* state_slots, int* last_token,
                                   int num_slots, int requests, const void* table, const void* pairs, int is_f32,
                                   float* out, int* resolved, int tokens, int hidden, int vocab, long long buckets,
                                   long long mul_prev, long long mul_cur, unsigned* status, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0 && buckets > 0 && requests >= 0,
                "pair_embedding: bad sizes T=%d H=%d V=%d buckets=%lld", tokens, hidden, vocab, buckets);
  VOSTI_REQUIRE(mul_prev >= 0 && mul_cur >= 0 && mul_prev < (1ll << 31) && mul_cur < (1ll << 31),
                "pair_embedding: the multipliers must be non-negative and below 2^31");
  if (tokens == 0) return VOSTI_OK;
  if (is_f32)
    vosti_launch(pair_embedding_kernel<float>, dim3(tokens), dim3(128), 0, stream, ids, source, values, positions, request_of,
                 cu_q, state_slots, (const int*)last_token, num_slots, (const float*)table, (const float*)pairs, out, resolved,
                 hidden, vocab, buckets, mul_prev, mul_cur, status);
  else
    vosti_launch(pair_embedding_kernel<bf16>, dim3(tokens), dim3(128), 0, stream, ids, source, values, positions, request_of,
                 cu_q, state_slots, (const int*)last_token, num_slots, (const bf16*)table, (const bf16*)pairs, out, resolved,
                 hidden, vocab, buckets, mul_prev, mul_cur, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { vosti_set_error("%s", cudaGetErrorString(e)); return (int)e; }
  // the slots are rewritten only after every token of the step has read the old ones
  vosti_launch(pair_state_kernel, dim3((requests + 127) / 128), dim3(128), 0, stream, (const int*)resolved, cu_q, state_slots,
               last_token, num_slots, requests);
  VOSTI_LAUNCH_CHECK();
}

// z, out [tokens, dim] in the serving type; side [vocab, side_stride] in its own type.
VOSTI_API int vosti_token_gate(const void* z, int is_f32, const int* ids, const void* side, int side_f32, int64_t side_stride,
                               int offset, int dim, int vocab, void* out, int tokens, cudaStream_t stream) {
  VOSTI_REQUIRE(tokens >= 0 && dim > 0 && vocab > 0 && offset >= 0 && offset + dim <= side_stride, "token_gate: bad sizes");
  if (tokens == 0) return VOSTI_OK;
  const int64_t n = (int64_t)tokens * dim;
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
#define VOSTI_GATE(T, TS)                                                                                              \
  vosti_launch(token_gate_kernel<T, TS>, dim3(blocks), dim3(256), 0, stream, (const T*)z, ids, (const TS*)side, side_stride, \
               offset, dim, vocab, (T*)out, (int64_t)tokens)
  if (is_f32 && side_f32) VOSTI_GATE(float, float);
  else if (is_f32) VOSTI_GATE(float, bf16);
  else if (side_f32) VOSTI_GATE(bf16, float);
  else VOSTI_GATE(bf16, bf16);
#undef VOSTI_GATE
  VOSTI_LAUNCH_CHECK();
}
