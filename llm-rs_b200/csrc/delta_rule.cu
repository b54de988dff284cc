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
// Two kernels and a small third:
//   prepare     a warp per (token, head), all tokens at once: decay, removal rate times unit key, unit key, and r, k, v
//               widened, as six float32 rows [tokens, heads * d];
//   recurrence  one block per (request, head, slice of 16 value columns) walks the request's tokens of the step in
//               order: a column of S depends on no other column, so the slices run side by side. Four adjacent lanes
//               share a column, each keeping a quarter of its key channels in registers; u^T S and S^T r are summed
//               over the four with two shuffles. The prepared rows come in chunks through two shared-memory buffers
//               (16-byte asynchronous copies), so the next chunk arrives while this one is walked, and are read as
//               16-byte broadcasts. The state lives in float32 per request slot, read at the start and written at the
//               end: a step of one token (decoding) and a prompt's portion are the same kernel;
//   output      a warp per (token, head): divides by the head's root mean square, applies the weight and the gate.
#include "common.cuh"
#include "mma_util.cuh"

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

constexpr int DR_COLS = 16, DR_LANES = 4, DR_THREADS = DR_COLS * DR_LANES;
enum { DR_W = 0, DR_AU = 1, DR_U = 2, DR_K = 3, DR_R = 4, DR_V = 5, DR_ROWS = 6 };

// prep: float32 [6][tokens][heads * d] in the order of the enum above.
template <typename TA>
__global__ void delta_prepare_kernel(const TA* __restrict__ r, const TA* __restrict__ k, const TA* __restrict__ v,
                                     const TA* __restrict__ a_raw, long long in_stride,
                                     const float* __restrict__ decay_raw, const float* __restrict__ decay_bias,
                                     const float* __restrict__ a_bias, float* __restrict__ prep, int n_tokens,
                                     int n_heads, int d, float decay_scale, float key_eps) {
  const int row = blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n_tokens * n_heads) return;
  const int t = row / n_heads, h = row % n_heads;
  const size_t in0 = (size_t)t * in_stride + (size_t)h * d, out0 = (size_t)t * n_heads * d + (size_t)h * d;
  const size_t plane = (size_t)n_tokens * n_heads * d;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float kv = to_float(k[in0 + i]);
    ss += kv * kv;
  }
  const float inv = 1.0f / sqrtf(warp_sum(ss) + key_eps);
  for (int i = lane; i < d; i += 32) {
    const float kv = to_float(k[in0 + i]), u = kv * inv;
    prep[DR_W * plane + out0 + i] = expf(-decay_scale * sigmoidf_(decay_raw[out0 + i] + decay_bias[h * d + i]));
    prep[DR_AU * plane + out0 + i] = sigmoidf_(to_float(a_raw[in0 + i]) + a_bias[h * d + i]) * u;
    prep[DR_U * plane + out0 + i] = u;
    prep[DR_K * plane + out0 + i] = kv;
    prep[DR_R * plane + out0 + i] = to_float(r[in0 + i]);
    prep[DR_V * plane + out0 + i] = to_float(v[in0 + i]);
  }
}

template <int DMAX>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const float* __restrict__ prep, float* __restrict__ state, const int* __restrict__ q_start,
                  const int* __restrict__ n_new, const int* __restrict__ slot_ids, float* __restrict__ o_raw,
                  int n_tokens, int n_heads, int d) {
  constexpr int CHUNK = DMAX >= 256 ? 4 : (DMAX >= 128 ? 8 : 16);
  constexpr int IPL = DMAX / DR_LANES;             // key channels per lane
  __shared__ __align__(16) float s_in[2][5][CHUNK][DMAX];      // W, AU, U, K, R of a chunk's tokens; channels >= d stay 0
  __shared__ __align__(16) float s_v[2][CHUNK][DR_COLS];
  const int req = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * DR_COLS;
  const int tid = threadIdx.x;
  const int col = col0 + tid / DR_LANES, part = tid % DR_LANES, i0 = part * IPL;
  const bool live = col < d;
  const int t0 = q_start[req], n = n_new[req];
  const int ch0 = head * d, width = n_heads * d;
  const size_t plane = (size_t)n_tokens * width;
  float* S_g = state + ((size_t)slot_ids[req] * n_heads + head) * d * d;
  float S[IPL];
#pragma unroll
  for (int i = 0; i < IPL; ++i) S[i] = (live && i0 + i < d) ? S_g[(size_t)(i0 + i) * d + col] : 0.f;
  for (int e = tid; e < 2 * 5 * CHUNK * DMAX; e += DR_THREADS) (&s_in[0][0][0][0])[e] = 0.f;
  for (int e = tid; e < 2 * CHUNK * DR_COLS; e += DR_THREADS) (&s_v[0][0][0])[e] = 0.f;
  __syncthreads();
  // 16-byte copies when every row starts on a 16-byte boundary, else element by element.
  const bool wide = d % 4 == 0;
  const int ncols = min(DR_COLS, d - col0);
  auto load_chunk = [&](int buf, int c0) {
    const int cn = min(CHUNK, n - c0);
    if (wide) {
      const int per_row = d / 4;
      for (int e = tid; e < 5 * cn * per_row; e += DR_THREADS) {
        const int a = e / (cn * per_row), rem = e % (cn * per_row), tt = rem / per_row, piece = rem % per_row;
        cp_async_16(&s_in[buf][a][tt][piece * 4], prep + a * plane + (size_t)(t0 + c0 + tt) * width + ch0 + piece * 4, 16);
      }
    } else {
      for (int e = tid; e < 5 * cn * d; e += DR_THREADS) {
        const int a = e / (cn * d), rem = e % (cn * d), tt = rem / d, i = rem % d;
        s_in[buf][a][tt][i] = prep[a * plane + (size_t)(t0 + c0 + tt) * width + ch0 + i];
      }
    }
    for (int e = tid; e < cn * ncols; e += DR_THREADS) {
      const int tt = e / ncols, c = e % ncols;
      s_v[buf][tt][c] = prep[DR_V * plane + (size_t)(t0 + c0 + tt) * width + ch0 + col0 + c];
    }
    cp_async_commit();
  };

  if (n > 0) load_chunk(0, 0);
  for (int c0 = 0, it = 0; c0 < n; c0 += CHUNK, ++it) {
    const int cn = min(CHUNK, n - c0), buf = it & 1;
    if (c0 + CHUNK < n) {
      load_chunk(buf ^ 1, c0 + CHUNK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
#pragma unroll 4
    for (int tt = 0; tt < cn; ++tt) {      // unrolled: the next tokens' rows are fetched under this token's shuffles
      const float vj = s_v[buf][tt][tid / DR_LANES];
      float us[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < IPL; i += 4) {
        const float4 u4 = *reinterpret_cast<const float4*>(&s_in[buf][DR_U][tt][i0 + i]);
        us[0] = fmaf(u4.x, S[i], us[0]);
        us[1] = fmaf(u4.y, S[i + 1], us[1]);
        us[2] = fmaf(u4.z, S[i + 2], us[2]);
        us[3] = fmaf(u4.w, S[i + 3], us[3]);
      }
      float uS = (us[0] + us[1]) + (us[2] + us[3]);
      uS += __shfl_xor_sync(0xffffffffu, uS, 1);
      uS += __shfl_xor_sync(0xffffffffu, uS, 2);
      float os[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < IPL; i += 4) {
        const float4 w4 = *reinterpret_cast<const float4*>(&s_in[buf][DR_W][tt][i0 + i]);
        const float4 a4 = *reinterpret_cast<const float4*>(&s_in[buf][DR_AU][tt][i0 + i]);
        const float4 k4 = *reinterpret_cast<const float4*>(&s_in[buf][DR_K][tt][i0 + i]);
        const float4 r4 = *reinterpret_cast<const float4*>(&s_in[buf][DR_R][tt][i0 + i]);
        S[i] = fmaf(k4.x, vj, fmaf(-a4.x, uS, w4.x * S[i]));
        S[i + 1] = fmaf(k4.y, vj, fmaf(-a4.y, uS, w4.y * S[i + 1]));
        S[i + 2] = fmaf(k4.z, vj, fmaf(-a4.z, uS, w4.z * S[i + 2]));
        S[i + 3] = fmaf(k4.w, vj, fmaf(-a4.w, uS, w4.w * S[i + 3]));
        os[0] = fmaf(S[i], r4.x, os[0]);
        os[1] = fmaf(S[i + 1], r4.y, os[1]);
        os[2] = fmaf(S[i + 2], r4.z, os[2]);
        os[3] = fmaf(S[i + 3], r4.w, os[3]);
      }
      float o = (os[0] + os[1]) + (os[2] + os[3]);
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (part == 0 && live) o_raw[(size_t)(t0 + c0 + tt) * width + ch0 + col] = o;
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
                        const int* q_start, const int* n_new, const int* slot_ids, float* work, void* out,
                        int n_tokens, int n_heads, int d, float decay_scale, float key_eps, float norm_eps) {
  const int rows = n_tokens * n_heads;
  float* prep = work;
  float* o_raw = work + (size_t)DR_ROWS * rows * d;
  delta_prepare_kernel<TA><<<(rows + 3) / 4, 128, 0, stream>>>((const TA*)r, (const TA*)k, (const TA*)v,
                                                               (const TA*)a_raw, in_stride, decay_raw, decay_bias,
                                                               a_bias, prep, n_tokens, n_heads, d, decay_scale, key_eps);
  int rc = llmrs_launch_status("delta_rule (prepare)");
  if (rc != 0) return rc;
  if (dmax == 32) delta_rule_kernel<32><<<grid, DR_THREADS, 0, stream>>>(prep, state, q_start, n_new, slot_ids, o_raw, n_tokens, n_heads, d);
  else if (dmax == 64) delta_rule_kernel<64><<<grid, DR_THREADS, 0, stream>>>(prep, state, q_start, n_new, slot_ids, o_raw, n_tokens, n_heads, d);
  else if (dmax == 128) delta_rule_kernel<128><<<grid, DR_THREADS, 0, stream>>>(prep, state, q_start, n_new, slot_ids, o_raw, n_tokens, n_heads, d);
  else delta_rule_kernel<256><<<grid, DR_THREADS, 0, stream>>>(prep, state, q_start, n_new, slot_ids, o_raw, n_tokens, n_heads, d);
  rc = llmrs_launch_status("delta_rule");
  if (rc != 0) return rc;
  delta_out_kernel<TA><<<(rows + 3) / 4, 128, 0, stream>>>(o_raw, (const TA*)gate, in_stride, norm_w, (TA*)out, rows,
                                                           n_heads, d, norm_eps);
  return llmrs_launch_status("delta_rule (norm and gate)");
}

// Float32 workspace the three kernels share, in floats.
LLMRS_API long long llmrs_delta_rule_work_floats(int n_tokens, int n_heads, int d) {
  return (long long)(DR_ROWS + 1) * n_tokens * n_heads * d;
}

// r, k, v, gate, a_raw: [tokens, ...] of the activation type, rows `in_stride` elements apart, each pointing at its
// own first column (head h's channels at h * d); decay_raw: float32 [tokens, heads * d]; work: float32 workspace of
// llmrs_delta_rule_work_floats, 16-byte aligned; out: [tokens, heads * d].
LLMRS_API int llmrs_delta_rule(const void* r, const void* k, const void* v, const void* gate, const void* a_raw,
                               long long in_stride, int dtype, const float* decay_raw, const float* decay_bias,
                               const float* a_bias, const float* norm_w, float* state, const int* q_start,
                               const int* n_new, const int* slot_ids, float* work, void* out, int n_tokens,
                               int n_requests, int n_heads, int d, float decay_scale, float key_eps, float norm_eps,
                               cudaStream_t stream) {
  LLMRS_REQUIRE(n_requests >= 0 && n_tokens >= 0 && n_heads > 0 && d > 0, "delta_rule: bad sizes");
  LLMRS_REQUIRE(d <= 256, "delta_rule: heads of at most 256 channels, got %d", d);
  LLMRS_REQUIRE(n_heads <= 65535, "delta_rule: too many heads");
  LLMRS_REQUIRE(((uintptr_t)work & 15) == 0, "delta_rule: the workspace must be 16-byte aligned");
  if (n_requests == 0 || n_tokens == 0) return 0;
  const int dmax = d <= 32 ? 32 : (d <= 64 ? 64 : (d <= 128 ? 128 : 256));
  dim3 grid(n_requests, n_heads, (d + DR_COLS - 1) / DR_COLS);
  if (dtype == LLMRS_F32)
    return launch_delta<float>(dmax, grid, stream, r, k, v, gate, a_raw, in_stride, decay_raw, decay_bias, a_bias,
                               norm_w, state, q_start, n_new, slot_ids, work, out, n_tokens, n_heads, d, decay_scale,
                               key_eps, norm_eps);
  if (dtype == LLMRS_BF16)
    return launch_delta<__nv_bfloat16>(dmax, grid, stream, r, k, v, gate, a_raw, in_stride, decay_raw, decay_bias,
                                       a_bias, norm_w, state, q_start, n_new, slot_ids, work, out, n_tokens, n_heads,
                                       d, decay_scale, key_eps, norm_eps);
  return llmrs_fail("delta_rule: unknown dtype %d", dtype);
}
