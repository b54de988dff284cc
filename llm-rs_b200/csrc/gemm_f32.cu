// True 32-bit matrix product for the float32 path: out[m, n] = sum_k x[m, k] * w[n, k] (+ bias[n]).
//
// FFMA on the CUDA cores, no tensor-core mode of reduced precision. Every output
// element is summed over k in the same order whatever M is, so a token's result does
// not depend on what else is in the batch. The reference's products are library calls
// (llm-core/src/backends/candle.rs:1276-1340: weight [out, in], used transposed,
// optional bias added after).
#include "common.cuh"

constexpr int GF_BM = 64, GF_BN = 64, GF_BK = 16, GF_THREADS = 256;

template <typename TX>
__global__ void __launch_bounds__(GF_THREADS)
gemm_f32_kernel(const TX* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                float* __restrict__ out, int M, int N, int K, long long x_stride, long long out_stride) {
  __shared__ float As[GF_BK][GF_BM + 4];
  __shared__ float Bs[GF_BK][GF_BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * GF_BM, n0 = blockIdx.x * GF_BN;
  const int tr = tid / 16, tc = tid % 16;  // this thread's 4x4 block: rows tr*4.., cols tc*4..
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // Each thread loads 4 consecutive k of one row of each tile.
  const int lrow = tid / 4, lk = (tid % 4) * 4;
  for (int k0 = 0; k0 < K; k0 += GF_BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int m = m0 + lrow, n = n0 + lrow;
      As[lk + e][lrow] = (m < M && k < K) ? to_float(x[(size_t)m * x_stride + k]) : 0.f;
      Bs[lk + e][lrow] = (n < N && k < K) ? w[(size_t)n * K + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GF_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][tr * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tc * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + tr * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tc * 4 + j;
      if (n < N) out[(size_t)m * out_stride + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
  }
}

LLMRS_API int llmrs_gemm_f32(const float* x, long long x_stride, const float* w, const float* bias, float* out,
                             long long out_stride, int M, int N, int K, cudaStream_t stream) {
  LLMRS_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_f32: bad sizes M=%d N=%d K=%d", M, N, K);
  if (M == 0) return 0;
  dim3 grid((N + GF_BN - 1) / GF_BN, (M + GF_BM - 1) / GF_BM);
  LLMRS_REQUIRE(grid.y <= 65535, "gemm_f32: M=%d is too large", M);
  gemm_f32_kernel<float><<<grid, GF_THREADS, 0, stream>>>(x, w, bias, out, M, N, K, x_stride, out_stride);
  return llmrs_launch_status("gemm_f32");
}

// The same product for rows stored in bfloat16 (activations of the bfloat16 path whose product must not be rounded:
// a router's logits, the gates of a recurrence): the rows are widened as they are read, weights, sums and output
// are float32.
LLMRS_API int llmrs_gemm_f32_bf16_rows(const void* x, long long x_stride, const float* w, const float* bias, float* out,
                                       long long out_stride, int M, int N, int K, cudaStream_t stream) {
  LLMRS_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_f32: bad sizes M=%d N=%d K=%d", M, N, K);
  if (M == 0) return 0;
  dim3 grid((N + GF_BN - 1) / GF_BN, (M + GF_BM - 1) / GF_BM);
  LLMRS_REQUIRE(grid.y <= 65535, "gemm_f32: M=%d is too large", M);
  gemm_f32_kernel<__nv_bfloat16><<<grid, GF_THREADS, 0, stream>>>((const __nv_bfloat16*)x, w, bias, out, M, N, K,
                                                                  x_stride, out_stride);
  return llmrs_launch_status("gemm_f32 (bfloat16 rows)");
}

// ---------------------------------------------------------------------------------
// Few output features (a router's logits, the gates of a recurrence, a single gate row): out[m, n] for n < N <= some
// hundreds. The tiled kernel above would run as one or two blocks that walk K alone; here a block holds SK_TOKENS
// rows of x in shared memory and each of its warps owns one output feature: its lanes walk that weight row once,
// four values per load, against all the block's rows. Every output is summed in the same order whatever M is (a
// lane's own values in order of k, then the lanes by butterfly), so a token's result does not depend on the batch.
// ---------------------------------------------------------------------------------
constexpr int SK_WARPS = 8, SK_THREADS = SK_WARPS * 32, SK_TOKENS = 8;

// SPLIT false: a warp owns a feature and walks all of K. SPLIT true (few rows: decoding): a block owns ONE feature,
// its warps walk an eighth of K each and the block adds the eight parts in warp order, so that a product of a
// handful of rows still fills the device.
template <typename TX, bool SPLIT>
__global__ void __launch_bounds__(SK_THREADS)
gemm_f32_skinny_kernel(const TX* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                       float* __restrict__ out, int M, int N, int K, long long x_stride, long long out_stride) {
  extern __shared__ __align__(16) unsigned char sk_raw[];
  __shared__ float parts[SK_WARPS][SK_TOKENS];
  TX* xs = reinterpret_cast<TX*>(sk_raw);      // [SK_TOKENS][K]
  const int m0 = blockIdx.x * SK_TOKENS, rows = min(SK_TOKENS, M - m0);
  for (int i = threadIdx.x; i < SK_TOKENS * K; i += SK_THREADS) {
    const int r = i / K, k = i - r * K;
    xs[i] = r < rows ? x[(size_t)(m0 + r) * x_stride + k] : TX(0.f);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = SPLIT ? (int)blockIdx.y : (int)blockIdx.y * SK_WARPS + warp;
  const bool live = n < N;
  const float* wr = w + (size_t)(live ? n : 0) * K;
  float acc[SK_TOKENS];
#pragma unroll
  for (int r = 0; r < SK_TOKENS; ++r) acc[r] = 0.f;
  const int K4 = K & ~3;
  // The piece of K this warp walks: all of it, or its eighth (in whole groups of 128).
  const int piece = SPLIT ? (((K4 + 127) / 128 + SK_WARPS - 1) / SK_WARPS) * 128 : K4;
  const int k_lo = SPLIT ? warp * piece : 0, k_hi = min(K4, k_lo + piece);
  if (live) {
    for (int k = k_lo + lane * 4; k < k_hi; k += 128) {
      const float4 wv = *reinterpret_cast<const float4*>(wr + k);
#pragma unroll
      for (int r = 0; r < SK_TOKENS; ++r) {
        const TX* xr = xs + r * K + k;
        acc[r] = fmaf(to_float(xr[0]), wv.x, acc[r]);
        acc[r] = fmaf(to_float(xr[1]), wv.y, acc[r]);
        acc[r] = fmaf(to_float(xr[2]), wv.z, acc[r]);
        acc[r] = fmaf(to_float(xr[3]), wv.w, acc[r]);
      }
    }
    if (!SPLIT || warp == SK_WARPS - 1)
      for (int k = K4 + lane; k < K; k += 32) {
#pragma unroll
        for (int r = 0; r < SK_TOKENS; ++r) acc[r] = fmaf(to_float(xs[r * K + k]), wr[k], acc[r]);
      }
  }
#pragma unroll
  for (int r = 0; r < SK_TOKENS; ++r) {
    const float s = warp_sum(acc[r]);
    if (SPLIT) {
      if (lane == 0) parts[warp][r] = s;
    } else if (lane == 0 && live && r < rows) {
      out[(size_t)(m0 + r) * out_stride + n] = s + (bias ? bias[n] : 0.f);
    }
  }
  if (SPLIT) {
    __syncthreads();
    if (threadIdx.x < rows && live) {
      float s = 0.f;
#pragma unroll
      for (int wv = 0; wv < SK_WARPS; ++wv) s += parts[wv][threadIdx.x];
      out[(size_t)(m0 + threadIdx.x) * out_stride + n] = s + (bias ? bias[n] : 0.f);
    }
  }
}

// x_dtype: LLMRS_F32 or LLMRS_BF16 rows; w (16-byte aligned rows: K % 4 == 0), bias and out float32.
LLMRS_API int llmrs_gemm_f32_skinny(const void* x, int x_dtype, long long x_stride, const float* w, const float* bias,
                                    float* out, long long out_stride, int M, int N, int K, cudaStream_t stream) {
  LLMRS_REQUIRE(M >= 0 && N > 0 && K > 0 && K % 4 == 0, "gemm_f32_skinny: bad sizes M=%d N=%d K=%d", M, N, K);
  LLMRS_REQUIRE(((uintptr_t)w & 15) == 0, "gemm_f32_skinny: the weights must be 16-byte aligned");
  if (M == 0) return 0;
  const size_t smem = (size_t)SK_TOKENS * K * (x_dtype == LLMRS_F32 ? 4 : 2);
  LLMRS_REQUIRE(smem <= 200 * 1024, "gemm_f32_skinny: rows of %d values are too long", K);
  const bool split = M <= 4 * SK_TOKENS;       // few rows: a block per feature
  dim3 grid((M + SK_TOKENS - 1) / SK_TOKENS, split ? N : (N + SK_WARPS - 1) / SK_WARPS);
  LLMRS_REQUIRE(grid.y <= 65535, "gemm_f32_skinny: N=%d is too large", N);
#define LLMRS_SK_LAUNCH(T, S)                                                                                         \
  do {                                                                                                                \
    static size_t configured = 48 * 1024;                                                                             \
    if (smem > configured) {                                                                                          \
      cudaError_t e = cudaFuncSetAttribute(gemm_f32_skinny_kernel<T, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                                \
      if (e != cudaSuccess) return llmrs_fail("gemm_f32_skinny: shared memory %zu: %s", smem, cudaGetErrorString(e)); \
      configured = smem;                                                                                              \
    }                                                                                                                 \
    gemm_f32_skinny_kernel<T, S><<<grid, SK_THREADS, smem, stream>>>((const T*)x, w, bias, out, M, N, K, x_stride,    \
                                                                     out_stride);                                     \
  } while (0)
  if (x_dtype == LLMRS_F32 && split) LLMRS_SK_LAUNCH(float, true);
  else if (x_dtype == LLMRS_F32) LLMRS_SK_LAUNCH(float, false);
  else if (x_dtype == LLMRS_BF16 && split) LLMRS_SK_LAUNCH(__nv_bfloat16, true);
  else if (x_dtype == LLMRS_BF16) LLMRS_SK_LAUNCH(__nv_bfloat16, false);
  else return llmrs_fail("gemm_f32_skinny: unknown dtype %d", x_dtype);
#undef LLMRS_SK_LAUNCH
  return llmrs_launch_status("gemm_f32_skinny");
}
