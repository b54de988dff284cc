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
// One block per (request, head, slice of 16 value columns) walks the request's tokens of the step in order: a column
// of S depends on no other column, so the slices run side by side. Four adjacent lanes share a column, each keeping
// a quarter of its key channels in registers; u^T S and S^T r are summed over the four with two shuffles. The tokens
// are staged through shared memory in chunks: decay, removal rate and unit key of a chunk are computed by all
// threads at once (float32), then the serial part reads them as 16-byte broadcasts. The state lives in float32 per
// request slot and is read at the start and written at the end: a step of one token (decoding) and a prompt's
// portion are the same kernel. The raw outputs go to a float32 buffer; a second kernel (one warp per token and head)
// divides by the head's root mean square and applies the weight and the gate.
#include "common.cuh"

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

constexpr int DR_COLS = 16, DR_LANES = 4, DR_THREADS = DR_COLS * DR_LANES;

template <typename TA, int DMAX>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const TA* __restrict__ r, const TA* __restrict__ k, const TA* __restrict__ v,
                  const TA* __restrict__ a_raw, long long in_stride, const float* __restrict__ decay_raw,
                  const float* __restrict__ decay_bias, const float* __restrict__ a_bias, float* __restrict__ state,
                  const int* __restrict__ q_start, const int* __restrict__ n_new, const int* __restrict__ slot_ids,
                  float* __restrict__ o_raw, int n_heads, int d, float decay_scale, float key_eps) {
  constexpr int CHUNK = DMAX >= 128 ? 8 : 16;
  constexpr int IPL = DMAX / DR_LANES;             // key channels per lane
  __shared__ __align__(16) float s_r[CHUNK][DMAX], s_k[CHUNK][DMAX], s_w[CHUNK][DMAX], s_au[CHUNK][DMAX],
      s_u[CHUNK][DMAX];
  __shared__ float s_v[CHUNK][DR_COLS];
  const int req = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * DR_COLS;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int col = col0 + tid / DR_LANES, part = tid % DR_LANES, i0 = part * IPL;
  const bool live = col < d;
  const int t0 = q_start[req], n = n_new[req];
  const int ch0 = head * d;
  float* S_g = state + ((size_t)slot_ids[req] * n_heads + head) * d * d;
  float S[IPL];
#pragma unroll
  for (int i = 0; i < IPL; ++i) S[i] = (live && i0 + i < d) ? S_g[(size_t)(i0 + i) * d + col] : 0.f;

  for (int c0 = 0; c0 < n; c0 += CHUNK) {
    const int cn = min(CHUNK, n - c0);
    for (int e = tid; e < cn * DMAX; e += DR_THREADS) {     // channels beyond d are zeros: they add nothing
      const int tt = e / DMAX, i = e % DMAX;
      float rv = 0.f, kv = 0.f, wv = 0.f, av = 0.f;
      if (i < d) {
        const size_t at = (size_t)(t0 + c0 + tt) * in_stride + ch0 + i;
        rv = to_float(r[at]);
        kv = to_float(k[at]);
        wv = expf(-decay_scale * sigmoidf_(decay_raw[(size_t)(t0 + c0 + tt) * (n_heads * d) + ch0 + i]
                                           + decay_bias[ch0 + i]));
        av = sigmoidf_(to_float(a_raw[at]) + a_bias[ch0 + i]);
      }
      s_r[tt][i] = rv, s_k[tt][i] = kv, s_w[tt][i] = wv, s_au[tt][i] = av;
    }
    for (int e = tid; e < cn * DR_COLS; e += DR_THREADS) {
      const int tt = e / DR_COLS, c = e % DR_COLS;
      s_v[tt][c] = col0 + c < d ? to_float(v[(size_t)(t0 + c0 + tt) * in_stride + ch0 + col0 + c]) : 0.f;
    }
    __syncthreads();
    for (int tt = warp; tt < cn; tt += DR_THREADS / 32) {      // unit keys: one warp per token
      float ss = 0.f;
      for (int i = lane; i < DMAX; i += 32) ss += s_k[tt][i] * s_k[tt][i];
      const float inv = 1.0f / sqrtf(warp_sum(ss) + key_eps);
      for (int i = lane; i < DMAX; i += 32) {
        const float u = s_k[tt][i] * inv;
        s_u[tt][i] = u;
        s_au[tt][i] *= u;
      }
    }
    __syncthreads();
    for (int tt = 0; tt < cn; ++tt) {
      const float vj = s_v[tt][tid / DR_LANES];
      float uS = 0.f;
#pragma unroll
      for (int i = 0; i < IPL; i += 4) {
        const float4 u4 = *reinterpret_cast<const float4*>(&s_u[tt][i0 + i]);
        uS = fmaf(u4.x, S[i], fmaf(u4.y, S[i + 1], fmaf(u4.z, S[i + 2], fmaf(u4.w, S[i + 3], uS))));
      }
      uS += __shfl_xor_sync(0xffffffffu, uS, 1);
      uS += __shfl_xor_sync(0xffffffffu, uS, 2);
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < IPL; i += 4) {
        const float4 w4 = *reinterpret_cast<const float4*>(&s_w[tt][i0 + i]);
        const float4 a4 = *reinterpret_cast<const float4*>(&s_au[tt][i0 + i]);
        const float4 k4 = *reinterpret_cast<const float4*>(&s_k[tt][i0 + i]);
        const float4 r4 = *reinterpret_cast<const float4*>(&s_r[tt][i0 + i]);
        S[i] = fmaf(k4.x, vj, fmaf(-a4.x, uS, w4.x * S[i]));
        S[i + 1] = fmaf(k4.y, vj, fmaf(-a4.y, uS, w4.y * S[i + 1]));
        S[i + 2] = fmaf(k4.z, vj, fmaf(-a4.z, uS, w4.z * S[i + 2]));
        S[i + 3] = fmaf(k4.w, vj, fmaf(-a4.w, uS, w4.w * S[i + 3]));
        o = fmaf(S[i], r4.x, fmaf(S[i + 1], r4.y, fmaf(S[i + 2], r4.z, fmaf(S[i + 3], r4.w, o))));
      }
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (part == 0 && live) o_raw[(size_t)(t0 + c0 + tt) * (n_heads * d) + ch0 + col] = o;
    }
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < IPL; ++i)
      if (i0 + i < d) S_g[(size_t)(i0 + i) * d + col] = S[i];
  }
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight[h, :] * sigmoid(gate[t, h, :]); a warp per (t, h).
template <typename TA>
__global__ void delta_out_kernel(const float* __restrict__ o_raw, const TA* __restrict__ gate, long long gate_stride,
                                 const float* __restrict__ norm_w, TA* __restrict__ out, int n_rows, int n_heads,
                                 int d, float eps) {
  const int row = blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const int t = row / n_heads, h = row % n_heads;
  const float* o = o_raw + (size_t)t * n_heads * d + (size_t)h * d;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) ss += o[i] * o[i];
  const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)d + eps);
  for (int i = lane; i < d; i += 32) {
    const float g = sigmoidf_(to_float(gate[(size_t)t * gate_stride + h * d + i]));
    out[(size_t)t * n_heads * d + (size_t)h * d + i] = from_float<TA>(o[i] * inv * norm_w[h * d + i] * g);
  }
}

template <typename TA>
static int launch_delta(int dmax, dim3 grid, cudaStream_t stream, const void* r, const void* k, const void* v,
                        const void* gate, const void* a_raw, long long in_stride, const float* decay_raw,
                        const float* decay_bias, const float* a_bias, const float* norm_w, float* state,
                        const int* q_start, const int* n_new, const int* slot_ids, float* o_raw, void* out,
                        int n_tokens, int n_heads, int d, float decay_scale, float key_eps, float norm_eps) {
#define LLMRS_DELTA(D)                                                                                             \
  delta_rule_kernel<TA, D><<<grid, DR_THREADS, 0, stream>>>((const TA*)r, (const TA*)k, (const TA*)v,              \
                                                            (const TA*)a_raw, in_stride, decay_raw, decay_bias,     \
                                                            a_bias, state, q_start, n_new, slot_ids, o_raw, n_heads, \
                                                            d, decay_scale, key_eps)
  if (dmax == 32) LLMRS_DELTA(32);
  else if (dmax == 64) LLMRS_DELTA(64);
  else if (dmax == 128) LLMRS_DELTA(128);
  else LLMRS_DELTA(256);
#undef LLMRS_DELTA
  int rc = llmrs_launch_status("delta_rule");
  if (rc != 0) return rc;
  const int rows = n_tokens * n_heads;
  delta_out_kernel<TA><<<(rows + 3) / 4, 128, 0, stream>>>(o_raw, (const TA*)gate, in_stride, norm_w, (TA*)out, rows,
                                                           n_heads, d, norm_eps);
  return llmrs_launch_status("delta_rule (norm and gate)");
}

// r, k, v, gate, a_raw: [tokens, ...] of the activation type, rows `in_stride` elements apart, each pointing at its
// own first column (head h's channels at h * d); decay_raw: float32 [tokens, heads * d]; o_raw: float32 workspace
// [tokens, heads * d]; out: [tokens, heads * d].
LLMRS_API int llmrs_delta_rule(const void* r, const void* k, const void* v, const void* gate, const void* a_raw,
                               long long in_stride, int dtype, const float* decay_raw, const float* decay_bias,
                               const float* a_bias, const float* norm_w, float* state, const int* q_start,
                               const int* n_new, const int* slot_ids, float* o_raw, void* out, int n_tokens,
                               int n_requests, int n_heads, int d, float decay_scale, float key_eps, float norm_eps,
                               cudaStream_t stream) {
  LLMRS_REQUIRE(n_requests >= 0 && n_tokens >= 0 && n_heads > 0 && d > 0, "delta_rule: bad sizes");
  LLMRS_REQUIRE(d <= 256, "delta_rule: heads of at most 256 channels, got %d", d);
  LLMRS_REQUIRE(n_heads <= 65535, "delta_rule: too many heads");
  if (n_requests == 0 || n_tokens == 0) return 0;
  const int dmax = d <= 32 ? 32 : (d <= 64 ? 64 : (d <= 128 ? 128 : 256));
  dim3 grid(n_requests, n_heads, (d + DR_COLS - 1) / DR_COLS);
  if (dtype == LLMRS_F32)
    return launch_delta<float>(dmax, grid, stream, r, k, v, gate, a_raw, in_stride, decay_raw, decay_bias, a_bias,
                               norm_w, state, q_start, n_new, slot_ids, o_raw, out, n_tokens, n_heads, d, decay_scale,
                               key_eps, norm_eps);
  if (dtype == LLMRS_BF16)
    return launch_delta<__nv_bfloat16>(dmax, grid, stream, r, k, v, gate, a_raw, in_stride, decay_raw, decay_bias,
                                       a_bias, norm_w, state, q_start, n_new, slot_ids, o_raw, out, n_tokens, n_heads,
                                       d, decay_scale, key_eps, norm_eps);
  return llmrs_fail("delta_rule: unknown dtype %d", dtype);
}
