// Linear recurrences with a matrix state per head, the common core of gated linear attention and matrix-memory
// recurrent layers:
//
//   S_t = a_t S_(t-1) + (b_t k_t) v_t^T        S: [key channel, value channel], float32, kept per request slot
//   o_t = S_t^T q_t
//
// with a scalar decay a_t and a scalar gain b_t per (token, head). A layer with a normaliser also carries
// n_t = a_t n_(t-1) + b_t k_t and divides o_t by max(|n_t . q_t|, floor_t) + den_eps: the normaliser is the state's
// column for a value that is always 1, and is computed as such.
//
// Kernels:
//   gate_scan    exponential gates with a running maximum m (m_t = max(f_t + m_(t-1), i_t), log-space input gate i and
//                forget gate f, both soft-capped): a warp per (request, head) scans the request's tokens of the step,
//                32 at a time, with the associative form of the (max, +) recurrence, and leaves
//                a_t = exp(f_t + m_(t-1) - m_t), b_t = exp(i_t - m_t), floor_t = exp(-m_t); m is kept per slot;
//   prepare      q, k, v of all tokens widened to float32 (optional SiLU, q scaled, k multiplied by its gain);
//   recurrence   a block per (request, head, 16 value columns) walks the tokens in order; four or eight adjacent lanes
//                share a column, each holding its part of the column's key channels in registers; rows arrive through two
//                shared-memory buffers by 16-byte asynchronous copies. A step of one token and a prompt's portion
//                are the same kernel;
//   output       divides by the normaliser, norms each head (or all heads together) by its root mean square,
//                multiplies by a weight and by sigmoid(gate), rounds to the activation type.
#include "common.cuh"
#include "mma_util.cuh"

__device__ __forceinline__ void cp_async_4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_addr(dst)), "l"(src));
}
__device__ __forceinline__ float lr_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float lr_logsigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// ---------------------------------------------------------------------------------
// gate_scan
// ---------------------------------------------------------------------------------
// gates: float32 [tokens, 2 * heads] (row stride given): the input gate's pre-activations, then the forget gate's.
__global__ void gate_scan_kernel(const float* __restrict__ gates, long long stride, float cap,
                                 float* __restrict__ m_state, const int* __restrict__ q_start,
                                 const int* __restrict__ n_new, const int* __restrict__ slot_ids,
                                 float* __restrict__ decay, float* __restrict__ gain, float* __restrict__ floor_,
                                 int n_heads) {
  const int req = blockIdx.x, lane = threadIdx.x & 31;
  const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (head >= n_heads) return;
  const int t0 = q_start[req], n = n_new[req];
  float* mp = m_state + (size_t)slot_ids[req] * n_heads + head;
  float m = *mp;
  for (int base = 0; base < n; base += 32) {
    const int t = base + lane;
    const bool live = t < n;
    // A lane without a token is the identity of the recurrence: m_out = max(0 + m_in, -inf).
    float f = 0.f, i = -INFINITY;
    if (live) {
      const float* g = gates + (size_t)(t0 + t) * stride;
      i = cap * tanhf(g[head] / cap);
      f = lr_logsigmoid(cap * tanhf(g[n_heads + head] / cap));
    }
    // Inclusive scan of (F, I) with m_out = max(F + m_in, I); later o earlier = (F_e + F_l, max(F_l + I_e, I_l)).
    float F = f, I = i;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float Fe = __shfl_up_sync(0xffffffffu, F, o), Ie = __shfl_up_sync(0xffffffffu, I, o);
      if (lane >= o) {
        I = fmaxf(F + Ie, I);
        F = Fe + F;
      }
    }
    const float m_t = fmaxf(F + m, I);
    float m_prev = __shfl_up_sync(0xffffffffu, m_t, 1);
    if (lane == 0) m_prev = m;
    if (live) {
      const size_t at = (size_t)(t0 + t) * n_heads + head;
      decay[at] = expf(f + m_prev - m_t);
      gain[at] = expf(i - m_t);
      floor_[at] = expf(-m_t);
    }
    m = __shfl_sync(0xffffffffu, m_t, 31);      // idle lanes carry the last token's value on
  }
  if (lane == 0) *mp = m;
}

LLMRS_API int llmrs_gate_scan(const float* gates, long long stride, float cap, float* m_state, const int* q_start,
                              const int* n_new, const int* slot_ids, float* decay, float* gain, float* floor_,
                              int n_requests, int n_heads, cudaStream_t stream) {
  LLMRS_REQUIRE(n_requests >= 0 && n_heads > 0 && cap > 0.f, "gate_scan: bad arguments");
  if (n_requests == 0) return 0;
  const int warps = n_heads < 4 ? n_heads : 4;
  dim3 grid(n_requests, (n_heads + warps - 1) / warps);
  gate_scan_kernel<<<grid, warps * 32, 0, stream>>>(gates, stride, cap, m_state, q_start, n_new, slot_ids, decay, gain,
                                                    floor_, n_heads);
  return llmrs_launch_status("gate_scan");
}

// ---------------------------------------------------------------------------------
// prepare: float32 planes Q [tokens, heads * dk], K [tokens, heads * dk], V [tokens, heads * dv]
// ---------------------------------------------------------------------------------
template <typename TA>
__global__ void lr_prepare_kernel(const TA* __restrict__ q, const TA* __restrict__ k, const TA* __restrict__ v,
                                  long long q_stride, long long k_stride, long long v_stride,
                                  const float* __restrict__ gain, float* __restrict__ Q, float* __restrict__ K,
                                  float* __restrict__ V, int n_heads, int dk, int dv, int act, float q_scale) {
  const int t = blockIdx.x;
  const int wk = n_heads * dk, wv = n_heads * dv;
  for (int c = threadIdx.x; c < wk; c += blockDim.x) {
    float qv = to_float(q[(size_t)t * q_stride + c]), kv = to_float(k[(size_t)t * k_stride + c]);
    if (act) {
      qv *= lr_sigmoid(qv);
      kv *= lr_sigmoid(kv);
    }
    Q[(size_t)t * wk + c] = qv * q_scale;
    K[(size_t)t * wk + c] = gain ? kv * gain[(size_t)t * n_heads + c / dk] : kv;
  }
  for (int c = threadIdx.x; c < wv; c += blockDim.x) {
    float vv = to_float(v[(size_t)t * v_stride + c]);
    if (act) vv *= lr_sigmoid(vv);
    V[(size_t)t * wv + c] = vv;
  }
}

// ---------------------------------------------------------------------------------
// recurrence
// ---------------------------------------------------------------------------------
constexpr int LR_COLS = 16;

// LR_LANES adjacent lanes share a column: 4 for heads of up to 64 key channels, 8 above (16 and 32 channels per lane
// instead of 32 and 64: shorter chains of dependent sums per token, and twice the warps on an SM that holds few blocks).
template <int DMAX, int LR_LANES>
__global__ void __launch_bounds__(LR_COLS * LR_LANES)
linear_recurrence_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                         const float* __restrict__ decay, const float* __restrict__ head_decay,
                         float* __restrict__ S_all, float* __restrict__ N_all, const int* __restrict__ q_start,
                         const int* __restrict__ n_new, const int* __restrict__ slot_ids, float* __restrict__ o_raw,
                         float* __restrict__ nq, int n_heads, int dk, int dv) {
  constexpr int CHUNK = DMAX >= 256 ? 8 : 16;
  constexpr int LR_THREADS = LR_COLS * LR_LANES;
  constexpr int IPL = DMAX / LR_LANES;             // key channels per lane
  __shared__ __align__(16) float s_q[2][CHUNK][DMAX];      // channels >= dk stay 0
  __shared__ __align__(16) float s_k[2][CHUNK][DMAX];
  __shared__ float s_v[2][CHUNK][LR_COLS];
  __shared__ float s_a[2][CHUNK];
  const int req = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * LR_COLS;
  const int tid = threadIdx.x;
  const int col = col0 + tid / LR_LANES, part = tid % LR_LANES;
  // A lane's channels come in groups of four, the groups of a column's lanes interleaved: register 4 g + e holds
  // channel g * 4 * LR_LANES + part * 4 + e, so that the lanes' 16-byte reads of a token's row lie side by side in
  // shared memory (a lane with one run of channels met its neighbours in the same banks).
  auto channel = [&](int i) { return (i >> 2) * 4 * LR_LANES + part * 4 + (i & 3); };
  const int n_cols = dv + (N_all != nullptr ? 1 : 0);      // the normaliser is one more column, whose value is 1
  const bool live = col < n_cols, is_norm = col == dv;
  const int t0 = q_start[req], n = n_new[req];
  const int wk = n_heads * dk, wv = n_heads * dv;
  const size_t slot = (size_t)slot_ids[req];
  float* S_g = S_all + (slot * n_heads + head) * (size_t)dk * dv;
  float* N_g = N_all ? N_all + (slot * n_heads + head) * (size_t)dk : nullptr;
  float S[IPL];
#pragma unroll
  for (int i = 0; i < IPL; ++i) {
    S[i] = 0.f;
    if (live && channel(i) < dk) S[i] = is_norm ? N_g[channel(i)] : S_g[(size_t)channel(i) * dv + col];
  }
  for (int e = tid; e < 2 * CHUNK * DMAX; e += LR_THREADS) {
    (&s_q[0][0][0])[e] = 0.f;
    (&s_k[0][0][0])[e] = 0.f;
  }
  __syncthreads();
  const bool wide = dk % 4 == 0;
  const float a_head = head_decay ? head_decay[head] : 1.0f;
  auto load_chunk = [&](int buf, int c0) {
    const int cn = min(CHUNK, n - c0);
    if (wide) {
      const int per_row = dk / 4;
      for (int e = tid; e < 2 * cn * per_row; e += LR_THREADS) {
        const int which = e / (cn * per_row), rem = e % (cn * per_row), tt = rem / per_row, piece = rem % per_row;
        const size_t src = (size_t)(t0 + c0 + tt) * wk + (size_t)head * dk + piece * 4;
        cp_async_16(which ? &s_k[buf][tt][piece * 4] : &s_q[buf][tt][piece * 4], (which ? K : Q) + src, 16);
      }
    } else {
      for (int e = tid; e < 2 * cn * dk; e += LR_THREADS) {
        const int which = e / (cn * dk), rem = e % (cn * dk), tt = rem / dk, i = rem % dk;
        const size_t src = (size_t)(t0 + c0 + tt) * wk + (size_t)head * dk + i;
        (which ? s_k : s_q)[buf][tt][i] = (which ? K : Q)[src];
      }
    }
    // Values and decays by 4-byte asynchronous copies too: a plain load would hold the warp for a memory round trip
    // at the top of every chunk, before it starts on the tokens it already has.
    for (int e = tid; e < cn * LR_COLS; e += LR_THREADS) {
      const int tt = e / LR_COLS, c = col0 + e % LR_COLS;
      if (c < dv) cp_async_4(&s_v[buf][tt][e % LR_COLS], V + (size_t)(t0 + c0 + tt) * wv + (size_t)head * dv + c);
      else s_v[buf][tt][e % LR_COLS] = 1.0f;
    }
    for (int tt = tid; tt < cn; tt += LR_THREADS) {
      if (decay) cp_async_4(&s_a[buf][tt], decay + (size_t)(t0 + c0 + tt) * n_heads + head);
      else s_a[buf][tt] = a_head;
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
    for (int tt = 0; tt < cn; ++tt) {
      const float vj = s_v[buf][tt][tid / LR_LANES], a = s_a[buf][tt];
      float os[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < IPL; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(&s_k[buf][tt][i * LR_LANES + part * 4]);
        const float4 q4 = *reinterpret_cast<const float4*>(&s_q[buf][tt][i * LR_LANES + part * 4]);
        S[i] = fmaf(k4.x, vj, a * S[i]);
        S[i + 1] = fmaf(k4.y, vj, a * S[i + 1]);
        S[i + 2] = fmaf(k4.z, vj, a * S[i + 2]);
        S[i + 3] = fmaf(k4.w, vj, a * S[i + 3]);
        os[0] = fmaf(S[i], q4.x, os[0]);
        os[1] = fmaf(S[i + 1], q4.y, os[1]);
        os[2] = fmaf(S[i + 2], q4.z, os[2]);
        os[3] = fmaf(S[i + 3], q4.w, os[3]);
      }
      float o = (os[0] + os[1]) + (os[2] + os[3]);
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (LR_LANES == 8) o += __shfl_xor_sync(0xffffffffu, o, 4);
      if (part == 0 && live) {
        if (is_norm) nq[(size_t)(t0 + c0 + tt) * n_heads + head] = o;
        else o_raw[(size_t)(t0 + c0 + tt) * wv + (size_t)head * dv + col] = o;
      }
    }
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < IPL; ++i)
      if (channel(i) < dk) {
        if (is_norm) N_g[channel(i)] = S[i];
        else S_g[(size_t)channel(i) * dv + col] = S[i];
      }
  }
}

// Floats of workspace for llmrs_linear_recurrence: the three prepared planes.
LLMRS_API long long llmrs_linear_recurrence_work_floats(int n_tokens, int n_heads, int dk, int dv) {
  return (long long)n_tokens * n_heads * (2LL * dk + dv) + 8;
}

// q, k, v: [tokens, ...] of the activation type with their row strides, head h's channels at h * dk (h * dv);
// act 1: SiLU on all three first; q is multiplied by q_scale; decay [tokens, heads] or null (then head_decay [heads],
// or 1 when that is null too); gain [tokens, heads] or null (1); S [slots, heads, dk, dv]; N [slots, heads, dk] or
// null (no normaliser: nq is not written); o_raw float32 [tokens, heads * dv]; nq float32 [tokens, heads].
LLMRS_API int llmrs_linear_recurrence(const void* q, const void* k, const void* v, long long q_stride,
                                      long long k_stride, long long v_stride, int dtype, int act, float q_scale,
                                      const float* decay, const float* head_decay, const float* gain, float* S,
                                      float* N, const int* q_start, const int* n_new, const int* slot_ids,
                                      float* work, float* o_raw, float* nq, int n_tokens, int n_requests, int n_heads,
                                      int dk, int dv, cudaStream_t stream) {
  LLMRS_REQUIRE(n_requests >= 0 && n_tokens >= 0 && n_heads > 0 && dk > 0 && dv > 0, "linear_recurrence: bad sizes");
  LLMRS_REQUIRE(dk <= 256, "linear_recurrence: heads of at most 256 key channels, got %d", dk);
  LLMRS_REQUIRE(n_heads <= 65535 && (dv + 16) / 16 <= 65535, "linear_recurrence: too many heads or columns");
  LLMRS_REQUIRE(((uintptr_t)work & 15) == 0, "linear_recurrence: the workspace must be 16-byte aligned");
  if (n_requests == 0 || n_tokens == 0) return 0;
  // Each plane starts on a 16-byte boundary.
  const size_t nk = ((size_t)n_tokens * n_heads * dk + 3) / 4 * 4;
  float* Q = work;
  float* K = Q + nk;
  float* V = K + nk;
  const int threads = n_heads * dk >= 1024 ? 256 : 128;
  if (dtype == LLMRS_F32)
    lr_prepare_kernel<float><<<n_tokens, threads, 0, stream>>>((const float*)q, (const float*)k, (const float*)v,
                                                               q_stride, k_stride, v_stride, gain, Q, K, V, n_heads,
                                                               dk, dv, act, q_scale);
  else if (dtype == LLMRS_BF16)
    lr_prepare_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, q_stride, k_stride, v_stride, gain,
        Q, K, V, n_heads, dk, dv, act, q_scale);
  else
    return llmrs_fail("linear_recurrence: unknown dtype %d", dtype);
  int rc = llmrs_launch_status("linear_recurrence (prepare)");
  if (rc != 0) return rc;
  const int cols = dv + (N != nullptr ? 1 : 0);
  dim3 grid(n_requests, n_heads, (cols + LR_COLS - 1) / LR_COLS);
#define LLMRS_LR_LAUNCH(D, L)                                                                                       \
  linear_recurrence_kernel<D, L><<<grid, LR_COLS * L, 0, stream>>>(Q, K, V, decay, head_decay, S, N, q_start, n_new, \
                                                                   slot_ids, o_raw, nq, n_heads, dk, dv)
  if (dk <= 32) LLMRS_LR_LAUNCH(32, 4);
  else if (dk <= 64) LLMRS_LR_LAUNCH(64, 4);
  else if (dk <= 128) LLMRS_LR_LAUNCH(128, 8);
  else LLMRS_LR_LAUNCH(256, 8);
#undef LLMRS_LR_LAUNCH
  return llmrs_launch_status("linear_recurrence");
}

// ---------------------------------------------------------------------------------
// output: out[t, h, :] = norm(o[t, h, :] / den[t, h]) * weight * sigmoid(gate[t, h, :]); one block per token.
// den = max(|nq|, floor) + den_eps when nq is given, else 1. per_head 1: each head is divided by its own root mean
// square; 0: all heads of a token together.
// ---------------------------------------------------------------------------------
template <typename TA>
__global__ void lr_output_kernel(const float* __restrict__ o_raw, const float* __restrict__ nq,
                                 const float* __restrict__ floor_, float den_eps, const TA* __restrict__ gate,
                                 long long gate_stride, const float* __restrict__ norm_w, TA* __restrict__ out,
                                 int n_heads, int dv, int per_head, float eps) {
  extern __shared__ float sh[];      // [heads] 1 / den, then [heads] sums of squares
  __shared__ float red[33];
  float* inv_den = sh;
  float* hss = sh + n_heads;
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  const float* o = o_raw + (size_t)t * n_heads * dv;
  for (int h = warp; h < n_heads; h += n_warps) {
    float id = 1.0f;
    if (nq) id = 1.0f / (fmaxf(fabsf(nq[(size_t)t * n_heads + h]), floor_[(size_t)t * n_heads + h]) + den_eps);
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) {
      const float x = o[h * dv + i] * id;
      ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) {
      inv_den[h] = id;
      hss[h] = ss;
    }
  }
  __syncthreads();
  float all = 0.f;
  if (!per_head) {
    float s = 0.f;
    for (int h = threadIdx.x; h < n_heads; h += blockDim.x) s += hss[h];
    all = 1.0f / sqrtf(block_sum(s, red) / (float)(n_heads * dv) + eps);
  }
  for (int c = threadIdx.x; c < n_heads * dv; c += blockDim.x) {
    const int h = c / dv;
    const float inv = per_head ? 1.0f / sqrtf(hss[h] / (float)dv + eps) : all;
    const float g = lr_sigmoid(to_float(gate[(size_t)t * gate_stride + c]));
    out[(size_t)t * n_heads * dv + c] = from_float<TA>(o[c] * inv_den[h] * inv * norm_w[c] * g);
  }
}

LLMRS_API int llmrs_recurrence_output(const float* o_raw, const float* nq, const float* floor_, float den_eps,
                                      const void* gate, long long gate_stride, int dtype, const float* norm_w,
                                      void* out, int n_tokens, int n_heads, int dv, int per_head, float eps,
                                      cudaStream_t stream) {
  LLMRS_REQUIRE(n_tokens >= 0 && n_heads > 0 && dv > 0 && n_heads <= 4096, "recurrence_output: bad sizes");
  LLMRS_REQUIRE((nq == nullptr) == (floor_ == nullptr), "recurrence_output: nq and floor come together");
  if (n_tokens == 0) return 0;
  const int threads = n_heads * dv >= 2048 ? 256 : 128;
  const size_t smem = 2 * (size_t)n_heads * sizeof(float);
  if (dtype == LLMRS_F32)
    lr_output_kernel<float><<<n_tokens, threads, smem, stream>>>(o_raw, nq, floor_, den_eps, (const float*)gate,
                                                                 gate_stride, norm_w, (float*)out, n_heads, dv,
                                                                 per_head, eps);
  else if (dtype == LLMRS_BF16)
    lr_output_kernel<__nv_bfloat16><<<n_tokens, threads, smem, stream>>>(
        o_raw, nq, floor_, den_eps, (const __nv_bfloat16*)gate, gate_stride, norm_w, (__nv_bfloat16*)out, n_heads, dv,
        per_head, eps);
  else
    return llmrs_fail("recurrence_output: unknown dtype %d", dtype);
  return llmrs_launch_status("recurrence_output");
}
