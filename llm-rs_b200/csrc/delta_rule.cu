// Generalized delta rule: a recurrent mixer whose per-head state S [key channel, value channel] is updated by
//
//   S <- diag(w) S - (a * u) (u^T S) + k v^T        (both products read the old S)
//   o  = S^T r
//
// with the unit key u = k / sqrt(sum(k^2) + key_eps), a per-channel decay w = exp(-decay_scale * sigmoid(d + d0))
// from the decay projection d, and a per-channel removal rate a = sigmoid(a_raw + a_bias). After the recurrence each
// head's o is divided by its root mean square, multiplied by a weight and by sigmoid(gate), and rounded to the
// activation type.
//
// One block per (request, head) walks the request's tokens of the step in order; thread j keeps column j of S in
// registers. The tokens are staged through shared memory in chunks: decay, removal rate and unit key of a chunk are
// computed by all threads at once (float32), then the serial part reads them as broadcasts. The state lives in
// float32 per request slot and is read at the start and written at the end: a step of one token (decoding) and a
// prompt's portion are the same kernel.
#include "common.cuh"

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename TA, int DMAX>
__global__ void __launch_bounds__(DMAX)
delta_rule_kernel(const TA* __restrict__ r, const TA* __restrict__ k, const TA* __restrict__ v,
                  const TA* __restrict__ gate, const TA* __restrict__ a_raw, long long in_stride,
                  const float* __restrict__ decay_raw, const float* __restrict__ decay_bias,
                  const float* __restrict__ a_bias, const float* __restrict__ norm_w, float* __restrict__ state,
                  const int* __restrict__ q_start, const int* __restrict__ n_new, const int* __restrict__ slot_ids,
                  TA* __restrict__ out, int n_heads, int d, float decay_scale, float key_eps, float norm_eps) {
  constexpr int CHUNK = DMAX >= 128 ? 8 : 16;
  constexpr int WARPS = DMAX / 32;
  __shared__ float s_r[CHUNK][DMAX], s_k[CHUNK][DMAX], s_v[CHUNK][DMAX];     // s_v is overwritten by o
  __shared__ float s_w[CHUNK][DMAX], s_au[CHUNK][DMAX], s_u[CHUNK][DMAX];
  __shared__ float s_inv[CHUNK];
  const int req = blockIdx.x, head = blockIdx.y;
  const int j = threadIdx.x, lane = j & 31, warp = j >> 5;
  const int t0 = q_start[req], n = n_new[req];
  const int col0 = head * d;
  float* S_g = state + ((size_t)slot_ids[req] * n_heads + head) * d * d;
  float S[DMAX];
#pragma unroll
  for (int i = 0; i < DMAX; ++i) S[i] = (i < d && j < d) ? S_g[(size_t)i * d + j] : 0.f;

  for (int c0 = 0; c0 < n; c0 += CHUNK) {
    const int cn = min(CHUNK, n - c0);
    // Stage the chunk: every thread takes elements (token, channel) in turn.
    for (int e = j; e < cn * d; e += DMAX) {
      const int tt = e / d, i = e % d;
      const size_t at = (size_t)(t0 + c0 + tt) * in_stride + col0 + i;
      s_r[tt][i] = to_float(r[at]);
      s_k[tt][i] = to_float(k[at]);
      s_v[tt][i] = to_float(v[at]);
      s_w[tt][i] = expf(-decay_scale * sigmoidf_(decay_raw[(size_t)(t0 + c0 + tt) * (n_heads * d) + col0 + i]
                                                 + decay_bias[col0 + i]));
      s_au[tt][i] = sigmoidf_(to_float(a_raw[at]) + a_bias[col0 + i]);
    }
    __syncthreads();
    for (int tt = warp; tt < cn; tt += WARPS) {      // unit keys: one warp per token
      float ss = 0.f;
      for (int i = lane; i < d; i += 32) ss += s_k[tt][i] * s_k[tt][i];
      const float inv = 1.0f / sqrtf(warp_sum(ss) + key_eps);
      for (int i = lane; i < d; i += 32) {
        const float u = s_k[tt][i] * inv;
        s_u[tt][i] = u;
        s_au[tt][i] *= u;
      }
    }
    __syncthreads();
    // The serial part: thread j owns column j of S.
    for (int tt = 0; tt < cn; ++tt) {
      const float vj = s_v[tt][j < d ? j : 0];
      float uS = 0.f;
#pragma unroll
      for (int i = 0; i < DMAX; ++i)
        if (i < d) uS = fmaf(s_u[tt][i], S[i], uS);
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < DMAX; ++i)
        if (i < d) {
          S[i] = fmaf(s_k[tt][i], vj, fmaf(-s_au[tt][i], uS, s_w[tt][i] * S[i]));
          o = fmaf(S[i], s_r[tt][i], o);
        }
      if (j < d) s_v[tt][j] = o;      // only thread j reads s_v[tt][j]
    }
    __syncthreads();
    for (int tt = warp; tt < cn; tt += WARPS) {      // each head's o over its root mean square
      float ss = 0.f;
      for (int i = lane; i < d; i += 32) ss += s_v[tt][i] * s_v[tt][i];
      const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)d + norm_eps);
      if (lane == 0) s_inv[tt] = inv;
    }
    __syncthreads();
    for (int e = j; e < cn * d; e += DMAX) {
      const int tt = e / d, i = e % d;
      const size_t t = (size_t)(t0 + c0 + tt);
      const float g = sigmoidf_(to_float(gate[t * in_stride + col0 + i]));
      out[t * (size_t)(n_heads * d) + col0 + i] = from_float<TA>(s_v[tt][i] * s_inv[tt] * norm_w[col0 + i] * g);
    }
    __syncthreads();
  }
  if (j < d) {
#pragma unroll
    for (int i = 0; i < DMAX; ++i)
      if (i < d) S_g[(size_t)i * d + j] = S[i];
  }
}

template <typename TA>
static int launch_delta(int dmax, dim3 grid, cudaStream_t stream, const void* r, const void* k, const void* v,
                        const void* gate, const void* a_raw, long long in_stride, const float* decay_raw,
                        const float* decay_bias, const float* a_bias, const float* norm_w, float* state,
                        const int* q_start, const int* n_new, const int* slot_ids, void* out, int n_heads, int d,
                        float decay_scale, float key_eps, float norm_eps) {
#define LLMRS_DELTA(D)                                                                                              \
  delta_rule_kernel<TA, D><<<grid, D, 0, stream>>>((const TA*)r, (const TA*)k, (const TA*)v, (const TA*)gate,       \
                                                    (const TA*)a_raw, in_stride, decay_raw, decay_bias, a_bias,     \
                                                    norm_w, state, q_start, n_new, slot_ids, (TA*)out, n_heads, d, \
                                                    decay_scale, key_eps, norm_eps)
  if (dmax == 32) LLMRS_DELTA(32);
  else if (dmax == 64) LLMRS_DELTA(64);
  else LLMRS_DELTA(128);
#undef LLMRS_DELTA
  return llmrs_launch_status("delta_rule");
}

// r, k, v, gate, a_raw: [tokens, ...] of the activation type, rows `in_stride` elements apart, each pointing at its
// own first column (head h's channels at h * d); decay_raw: float32 [tokens, heads * d]; out: [tokens, heads * d].
LLMRS_API int llmrs_delta_rule(const void* r, const void* k, const void* v, const void* gate, const void* a_raw,
                               long long in_stride, int dtype, const float* decay_raw, const float* decay_bias,
                               const float* a_bias, const float* norm_w, float* state, const int* q_start,
                               const int* n_new, const int* slot_ids, void* out, int n_requests, int n_heads, int d,
                               float decay_scale, float key_eps, float norm_eps, cudaStream_t stream) {
  LLMRS_REQUIRE(n_requests >= 0 && n_heads > 0 && d > 0, "delta_rule: bad sizes");
  LLMRS_REQUIRE(d <= 128, "delta_rule: heads of at most 128 channels, got %d", d);
  LLMRS_REQUIRE(n_heads <= 65535, "delta_rule: too many heads");
  if (n_requests == 0) return 0;
  const int dmax = d <= 32 ? 32 : (d <= 64 ? 64 : 128);
  dim3 grid(n_requests, n_heads);
  if (dtype == LLMRS_F32)
    return launch_delta<float>(dmax, grid, stream, r, k, v, gate, a_raw, in_stride, decay_raw, decay_bias, a_bias,
                               norm_w, state, q_start, n_new, slot_ids, out, n_heads, d, decay_scale, key_eps,
                               norm_eps);
  if (dtype == LLMRS_BF16)
    return launch_delta<__nv_bfloat16>(dmax, grid, stream, r, k, v, gate, a_raw, in_stride, decay_raw, decay_bias,
                                       a_bias, norm_w, state, q_start, n_new, slot_ids, out, n_heads, d, decay_scale,
                                       key_eps, norm_eps);
  return llmrs_fail("delta_rule: unknown dtype %d", dtype);
}
