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
#include "mma_util.cuh"

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
  int tile_rows;            // grouped mode: the most rows a tile of the list has (64 or 128)
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
  if (a.tiles != nullptr) {      // a tile of the list may hold more rows than this kernel's: several blocks share it
    const int pieces = a.tile_rows / GG_BM, tile = blockIdx.y / pieces, piece = blockIdx.y % pieces;
    if (tile >= *a.n_tiles) return;
    group = a.tiles[3 * tile], m0 = a.tiles[3 * tile + 1] + GG_BM * piece;
    rows = min(GG_BM, a.tiles[3 * tile + 2] - GG_BM * piece);
    if (rows <= 0) return;
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

// ---------------------------------------------------------------------------------
// The same products on the tensor cores for bfloat16 operands (mma.sync m16n8k16, float32 accumulators): tiles of
// 64 or 128 rows x 128 columns (64 of each product for the gated unit), k in steps of 32 through a double buffer of 16-byte asynchronous copies. Eight warps as
// 2 x 4, each 32 or 64 rows x 32 (or 2 x 16) columns. Shared rows are 40 elements apart, which
// spreads the fragments' 32-bit reads over all banks. A row's sums run over k in the same order whichever rows
// share its tile. Needs K % 8 == 0 and 16-byte aligned rows of X and W.
// ---------------------------------------------------------------------------------
constexpr int GM_BK = 32, GM_LD = GM_BK + 8, GM_THREADS = 256;
// Columns of a tile: 128, or 64 of each of the two products of the gated unit (the same shared memory either way).
template <bool GLU> struct GmCols { static constexpr int value = GLU ? 64 : 128; };

template <typename TO, bool GLU, int MT>      // MT: 16-row pieces per warp; the tile has 32 * MT rows
__global__ void __launch_bounds__(GM_THREADS) gemm_grouped_mma_kernel(const GroupedGemmArgs a) {
  constexpr int GM_BM = 32 * MT;
  constexpr int GM_BN = GmCols<GLU>::value, NT = GM_BN / 32;      // NT: 8-column pieces per warp
  __shared__ __align__(16) __nv_bfloat16 As[2][GM_BM][GM_LD];
  __shared__ __align__(16) __nv_bfloat16 Bs[2][GM_BN][GM_LD];
  __shared__ __align__(16) __nv_bfloat16 B2s[GLU ? 2 : 1][GLU ? GM_BN : 1][GM_LD];
  __shared__ long long row_off[GM_BM];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int group, m0, rows;
  if (a.tiles != nullptr) {
    if ((int)blockIdx.y >= *a.n_tiles) return;
    group = a.tiles[3 * blockIdx.y], m0 = a.tiles[3 * blockIdx.y + 1], rows = a.tiles[3 * blockIdx.y + 2];
  } else {
    group = blockIdx.z, m0 = blockIdx.y * GM_BM, rows = min(GM_BM, a.M - m0);
  }
  if (tid < GM_BM) {
    long long off = -1;
    if (tid < rows) {
      const int row = m0 + tid;
      off = (long long)(a.src ? a.src[row] : row) * a.x_stride + (a.tiles ? 0 : (long long)group * a.x_batch);
    }
    row_off[tid] = off;
  }
  __syncthreads();
  const __nv_bfloat16* x = (const __nv_bfloat16*)a.x;
  const __nv_bfloat16* w = (const __nv_bfloat16*)a.w + (size_t)group * a.w_batch;
  const __nv_bfloat16* w2 = GLU ? (const __nv_bfloat16*)a.w2 + (size_t)group * a.w_batch : nullptr;
  const int n0 = blockIdx.x * GM_BN;

  // Copies of one k step: rows x 4 pieces of 8 elements; a thread takes rows tid / 4, tid / 4 + 64, ...
  const int a_row = tid >> 2, piece = (tid & 3) * 8;
  long long a_off[GM_BM / 64];
#pragma unroll
  for (int h = 0; h < GM_BM / 64; ++h) a_off[h] = row_off[a_row + 64 * h];
  auto issue = [&](int stage, int k0) {
    const int k = k0 + piece;
    const int kb = k < a.K ? min(16, (a.K - k) * 2) : 0;      // bytes of this piece inside K (K % 8 == 0: 0 or 16)
#pragma unroll
    for (int h = 0; h < GM_BM / 64; ++h)
      cp_async_16(&As[stage][a_row + 64 * h][piece], x + (a_off[h] >= 0 ? a_off[h] : 0) + (kb ? k : 0),
                  a_off[h] >= 0 ? kb : 0);
#pragma unroll
    for (int h = 0; h < GM_BN / 64; ++h) {
      const int r = a_row + 64 * h, n = n0 + r;
      const bool in = n < a.N;
      cp_async_16(&Bs[stage][r][piece], w + (in ? (size_t)n * a.K : 0) + (kb ? k : 0), in ? kb : 0);
      if (GLU) cp_async_16(&B2s[stage][r][piece], w2 + (in ? (size_t)n * a.K : 0) + (kb ? k : 0), in ? kb : 0);
    }
    cp_async_commit();
  };

  const int wm = (warp >> 2) * (16 * MT), wn = (warp & 3) * (8 * NT);
  const int g = lane >> 2, t = lane & 3;
  float acc[MT][NT][4], acc2[GLU ? MT : 1][GLU ? NT : 1][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[i][j][e] = 0.f;
        if (GLU) acc2[i][j][e] = 0.f;
      }
  const int k_steps = (a.K + GM_BK - 1) / GM_BK;
  issue(0, 0);
  for (int ks = 0; ks < k_steps; ++ks) {
    const int stage = ks & 1;
    if (ks + 1 < k_steps) {
      issue(stage ^ 1, (ks + 1) * GM_BK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // Fragments come by ldmatrix: lane l gives the address of row l % 8 of 8 x 8 piece l / 8.
    const int lm = lane >> 3, lr = lane & 7;
#pragma unroll
    for (int kk = 0; kk < GM_BK; kk += 16) {
      uint32_t af[MT][4];
#pragma unroll
      for (int i = 0; i < MT; ++i)     // pieces: rows 0-7 / 8-15 at k 0-7, then the same at k 8-15
        ldmatrix_x4(af[i], &As[stage][wm + 16 * i + (lm & 1) * 8 + lr][kk + (lm >> 1) * 8]);
#pragma unroll
      for (int j = 0; j < NT; j += 2) {
        uint32_t b[4];                 // pieces: columns j at k 0-7 / 8-15, then columns j + 1
        ldmatrix_x4(b, &Bs[stage][wn + 8 * (j + (lm >> 1)) + lr][kk + (lm & 1) * 8]);
#pragma unroll
        for (int i = 0; i < MT; ++i) {
          mma_bf16_16816(acc[i][j], af[i], b[0], b[1]);
          mma_bf16_16816(acc[i][j + 1], af[i], b[2], b[3]);
        }
        if (GLU) {
          uint32_t c[4];
          ldmatrix_x4(c, &B2s[stage][wn + 8 * (j + (lm >> 1)) + lr][kk + (lm & 1) * 8]);
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            mma_bf16_16816(acc2[i][j], af[i], c[0], c[1]);
            mma_bf16_16816(acc2[i][j + 1], af[i], c[2], c[3]);
          }
        }
      }
    }
    __syncthreads();
  }
  TO* out = (TO*)a.out + (a.tiles ? 0 : (size_t)group * a.out_batch);
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm + 16 * i + g + 8 * half;
      if (r >= rows) continue;
      TO* o = out + (size_t)(m0 + r) * a.out_stride;
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int n = n0 + wn + 8 * j + 2 * t + e;
          if (n >= a.N) continue;
          float v = acc[i][j][2 * half + e];
          if (GLU) {
            const float gt = fminf(v, a.limit);
            const float u = fminf(fmaxf(acc2[i][j][2 * half + e], -a.limit), a.limit);
            v = gt * (1.0f / (1.0f + expf(-a.alpha * gt))) * (u + a.shift);
          }
          o[n] = from_float<TO>(v);
        }
    }
}

template <typename TO, int MT>
static int launch_grouped_mma(const GroupedGemmArgs& a, dim3 grid, cudaStream_t stream) {
  if (a.w2 != nullptr)
    gemm_grouped_mma_kernel<TO, true, MT><<<grid, GM_THREADS, 0, stream>>>(a);
  else
    gemm_grouped_mma_kernel<TO, false, MT><<<grid, GM_THREADS, 0, stream>>>(a);
  return llmrs_launch_status("gemm_grouped (tensor cores)");
}

// 0: the CUDA-core kernel for every product (set by tests that compare the two).
static int g_grouped_mma = 1;
LLMRS_API void llmrs_gemm_grouped_use_mma(int on) { g_grouped_mma = on; }

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
                                 const int* tiles, const int* n_tiles, int max_tiles, int tile_rows, const int* src,
                                 int round_x, float limit, float alpha, float shift, cudaStream_t stream) {
  LLMRS_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_grouped: bad sizes M=%d N=%d K=%d", M, N, K);
  LLMRS_REQUIRE((tiles != nullptr) != (batches > 0), "gemm_grouped: either a tile list or a number of batches");
  LLMRS_REQUIRE(tiles == nullptr || n_tiles != nullptr, "gemm_grouped: a tile list needs its length");
  LLMRS_REQUIRE(tiles == nullptr || tile_rows == 64 || tile_rows == 128, "gemm_grouped: tiles of 64 or 128 rows");
  if (tiles == nullptr) tile_rows = M >= 128 ? 128 : 64;      // batched mode: the rows are cut here
  if (M == 0) return 0;
  GroupedGemmArgs a;
  a.x = x, a.x_stride = x_stride, a.x_batch = x_batch, a.w = w, a.w2 = w2, a.w_batch = w_batch;
  a.out = out, a.out_stride = out_stride, a.out_batch = out_batch, a.M = M, a.N = N, a.K = K;
  a.tiles = tiles, a.n_tiles = n_tiles, a.src = src, a.round_x = round_x, a.tile_rows = tile_rows;
  a.limit = limit, a.alpha = alpha, a.shift = shift;
  dim3 grid((N + GG_BN - 1) / GG_BN, tiles ? max_tiles * (tile_rows / GG_BM) : (M + GG_BM - 1) / GG_BM,
            tiles ? 1 : batches);
  LLMRS_REQUIRE(grid.y >= 1 && grid.y <= 65535 && grid.z <= 65535, "gemm_grouped: too many tiles or batches");
  // bfloat16 operands whose rows can be copied 16 bytes at a time go to the tensor cores.
  if (g_grouped_mma && x_dtype == LLMRS_BF16 && w_dtype == LLMRS_BF16 && K % 8 == 0 && x_stride % 8 == 0 &&
      x_batch % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && (!w2 || ((uintptr_t)w2 & 15) == 0) &&
      (N * (long long)K) % 8 == 0) {
    const int cols = w2 ? GmCols<true>::value : GmCols<false>::value;
    dim3 mgrid((N + cols - 1) / cols, tiles ? max_tiles : (M + tile_rows - 1) / tile_rows, grid.z);
    if (tile_rows == 128)
      return out_dtype == LLMRS_BF16 ? launch_grouped_mma<__nv_bfloat16, 4>(a, mgrid, stream)
                                     : launch_grouped_mma<float, 4>(a, mgrid, stream);
    return out_dtype == LLMRS_BF16 ? launch_grouped_mma<__nv_bfloat16, 2>(a, mgrid, stream)
                                   : launch_grouped_mma<float, 2>(a, mgrid, stream);
  }
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
