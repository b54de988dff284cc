// Many small matrix products in one launch: out[row, n] = sum_k X[src(row), k] * W_g[n, k], every product g with a
// weight matrix of its own ([N, K] row-major, `w_batch` elements apart).
//
//   batched   g = blockIdx.z; all products have the same M rows. Rows, batches and outputs have strides, so the
//             heads of a [tokens, heads, dim] tensor are batches without a copy.
//   grouped   the rows are sorted by group (expert) beforehand; a device-side list of tiles (group, first row, rows)
//             says which rows belong to which weights, `src` maps a sorted row to the row of X it reads.
//
// Epilogues: store, or the gated unit y = g * sigmoid(alpha * g) * (u + shift) with g = min(gate, limit) and
// u = clamp(up, -limit, limit), gate and up being two products over the same rows (weights `w` and `w2`).
//
// CUDA cores with float32 accumulation in a fixed order over k: a row's result does not depend on which rows share its
// tile. bfloat16 operands are widened exactly; with `round_x` float32 rows of X are first rounded to bfloat16 (they
// stand in for activations of that type).
#include "common.cuh"

constexpr int GG_BM = 64, GG_BN = 64, GG_BK = 16, GG_THREADS = 256;

struct GroupedGemmArgs {
  const void* x;            // rows of X
  long long x_stride;       // elements between rows
  long long x_batch;        // elements between batches (batched mode)
  const void* w;            // [groups, N, K]
  const void* w2;           // second weights of the gated unit, or null
  long long w_batch;        // elements between groups
  void* out;
  long long out_stride, out_batch;
  int M, N, K;              // M: rows (batched mode) or total sorted rows (grouped mode)
  const int* tiles;         // grouped mode: [tile][3] = group, first row, rows; null in batched mode
  const int* n_tiles;       // grouped mode: number of tiles on the device
  const int* src;           // grouped mode: sorted row -> row of X (null: the row itself)
  int round_x;
  float limit, alpha, shift;
};

template <typename T> __device__ __forceinline__ float load_as_float(const T* p, int round_bf16);
template <> __device__ __forceinline__ float load_as_float<float>(const float* p, int round_bf16) {
  const float v = *p;
  return round_bf16 ? __bfloat162float(__float2bfloat16_rn(v)) : v;
}
template <> __device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p, int) {
  return __bfloat162float(*p);
}

template <typename TX, typename TW, typename TO, bool GLU>
__global__ void __launch_bounds__(GG_THREADS) gemm_grouped_kernel(const GroupedGemmArgs a) {
  __shared__ float As[GG_BK][GG_BM + 4];
  __shared__ float Bs[GG_BK][GG_BN + 4];
  __shared__ float B2s[GLU ? GG_BK : 1][GG_BN + 4];
  __shared__ long long row_off[GG_BM];      // element offset of each tile row in X, -1: no such row

  const int tid = threadIdx.x;
  int group, m0, rows;
  if (a.tiles != nullptr) {
    if ((int)blockIdx.y >= *a.n_tiles) return;
    group = a.tiles[3 * blockIdx.y], m0 = a.tiles[3 * blockIdx.y + 1], rows = a.tiles[3 * blockIdx.y + 2];
  } else {
    group = blockIdx.z, m0 = blockIdx.y * GG_BM, rows = min(GG_BM, a.M - m0);
  }
  if (tid < GG_BM) {
    long long off = -1;
    if (tid < rows) {
      const int row = m0 + tid;
      off = (long long)(a.src ? a.src[row] : row) * a.x_stride + (a.tiles ? 0 : (long long)group * a.x_batch);
    }
    row_off[tid] = off;
  }
  __syncthreads();
  const TX* x = (const TX*)a.x;
  const TW* w = (const TW*)a.w + (size_t)group * a.w_batch;
  const TW* w2 = GLU ? (const TW*)a.w2 + (size_t)group * a.w_batch : nullptr;
  const int n0 = blockIdx.x * GG_BN;
  const int tr = tid / 16, tc = tid % 16;
  float acc[4][4], acc2[GLU ? 4 : 1][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[i][j] = 0.f;
      if (GLU) acc2[i][j] = 0.f;
    }
  const int lrow = tid / 4, lk = (tid % 4) * 4;
  const long long xo = row_off[lrow];
  const int n_l = n0 + lrow;
  for (int k0 = 0; k0 < a.K; k0 += GG_BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const bool kin = k < a.K;
      As[lk + e][lrow] = (xo >= 0 && kin) ? load_as_float<TX>(x + xo + k, a.round_x) : 0.f;
      Bs[lk + e][lrow] = (n_l < a.N && kin) ? to_float(w[(size_t)n_l * a.K + k]) : 0.f;
      if (GLU) B2s[lk + e][lrow] = (n_l < a.N && kin) ? to_float(w2[(size_t)n_l * a.K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GG_BK; ++kk) {
      float av[4], bv[4], b2v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][tr * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        bv[j] = Bs[kk][tc * 4 + j];
        if (GLU) b2v[j] = B2s[kk][tc * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
          if (GLU) acc2[i][j] = fmaf(av[i], b2v[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }
  TO* out = (TO*)a.out + (a.tiles ? 0 : (size_t)group * a.out_batch);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = tr * 4 + i;
    if (r >= rows) continue;
    TO* o = out + (size_t)(m0 + r) * a.out_stride;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tc * 4 + j;
      if (n >= a.N) continue;
      float v = acc[i][j];
      if (GLU) {
        const float g = fminf(v, a.limit);
        const float u = fminf(fmaxf(acc2[i][j], -a.limit), a.limit);
        v = g * (1.0f / (1.0f + expf(-a.alpha * g))) * (u + a.shift);
      }
      o[n] = from_float<TO>(v);
    }
  }
}

template <typename TX, typename TW, typename TO>
static int launch_grouped(const GroupedGemmArgs& a, dim3 grid, cudaStream_t stream) {
  if (a.w2 != nullptr)
    gemm_grouped_kernel<TX, TW, TO, true><<<grid, GG_THREADS, 0, stream>>>(a);
  else
    gemm_grouped_kernel<TX, TW, TO, false><<<grid, GG_THREADS, 0, stream>>>(a);
  return llmrs_launch_status("gemm_grouped");
}

// Types: x_dtype / w_dtype / out_dtype are LLMRS_F32 or LLMRS_BF16. Supported: all float32; bfloat16 weights with
// X in either type and the output in either type. `batches` > 0: batched mode; `tiles` != null: grouped mode with at
// most `max_tiles` tiles.
LLMRS_API int llmrs_gemm_grouped(const void* x, int x_dtype, long long x_stride, long long x_batch, const void* w,
                                 const void* w2, int w_dtype, long long w_batch, void* out, int out_dtype,
                                 long long out_stride, long long out_batch, int M, int N, int K, int batches,
                                 const int* tiles, const int* n_tiles, int max_tiles, const int* src, int round_x,
                                 float limit, float alpha, float shift, cudaStream_t stream) {
  LLMRS_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_grouped: bad sizes M=%d N=%d K=%d", M, N, K);
  LLMRS_REQUIRE((tiles != nullptr) != (batches > 0), "gemm_grouped: either a tile list or a number of batches");
  LLMRS_REQUIRE(tiles == nullptr || n_tiles != nullptr, "gemm_grouped: a tile list needs its length");
  if (M == 0) return 0;
  GroupedGemmArgs a;
  a.x = x, a.x_stride = x_stride, a.x_batch = x_batch, a.w = w, a.w2 = w2, a.w_batch = w_batch;
  a.out = out, a.out_stride = out_stride, a.out_batch = out_batch, a.M = M, a.N = N, a.K = K;
  a.tiles = tiles, a.n_tiles = n_tiles, a.src = src, a.round_x = round_x;
  a.limit = limit, a.alpha = alpha, a.shift = shift;
  dim3 grid((N + GG_BN - 1) / GG_BN, tiles ? max_tiles : (M + GG_BM - 1) / GG_BM, tiles ? 1 : batches);
  LLMRS_REQUIRE(grid.y >= 1 && grid.y <= 65535 && grid.z <= 65535, "gemm_grouped: too many tiles or batches");
  const int key = x_dtype * 4 + w_dtype * 2 + out_dtype;
  switch (key) {
    case 0: return launch_grouped<float, float, float>(a, grid, stream);
    case 2: return launch_grouped<float, __nv_bfloat16, float>(a, grid, stream);
    case 3: return launch_grouped<float, __nv_bfloat16, __nv_bfloat16>(a, grid, stream);
    case 6: return launch_grouped<__nv_bfloat16, __nv_bfloat16, float>(a, grid, stream);
    case 7: return launch_grouped<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(a, grid, stream);
    default: return llmrs_fail("gemm_grouped: unsupported types x=%d w=%d out=%d", x_dtype, w_dtype, out_dtype);
  }
}
