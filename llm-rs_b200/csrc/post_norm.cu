// Blocks whose norm comes AFTER the residual sum, and the small element-wise kernels such designs use.
//
//   post_norm   h[t] = rms(alpha * h[t] + y[t] * ls) * w, in place on the float32 residual stream, one block per
//               row; the same pass can also leave the row rounded to the activation type, which is what the next
//               branch's products read. `ls` (a per-channel scale of the branch) and `y` may be null.
//   relu_sq     out = max(x, 0)^2
//   scale       z *= s, float32, in place (a head whose logits are scaled)
//
// Sums, statistics and the normed value are float32; one rounding at the end.
#include "common.cuh"

template <typename TY, typename TO>
__global__ void post_norm_kernel(float* __restrict__ h, const TY* __restrict__ y, const float* __restrict__ ls,
                                 const float* __restrict__ w, TO* __restrict__ out, int width, float alpha, float eps) {
  extern __shared__ float row[];       // the summed row, kept between the two passes
  __shared__ float red[33];
  float* hr = h + (size_t)blockIdx.x * width;
  const TY* yr = y ? y + (size_t)blockIdx.x * width : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = alpha * hr[c];
    if (yr) v = fmaf(to_float(yr[c]), ls ? ls[c] : 1.0f, v);
    row[c] = v;
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = row[c] * inv * w[c];
    hr[c] = v;
    if (out) out[(size_t)blockIdx.x * width + c] = from_float<TO>(v);
  }
}

template <typename TY>
static int launch_post_norm(float* h, const void* y, const float* ls, const float* w, void* out, int out_dtype,
                            int n_rows, int width, float alpha, float eps, cudaStream_t stream) {
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  const size_t smem = (size_t)width * sizeof(float);
  if (out == nullptr || out_dtype == LLMRS_F32)
    post_norm_kernel<TY, float><<<n_rows, threads, smem, stream>>>(h, (const TY*)y, ls, w, (float*)out, width, alpha, eps);
  else if (out_dtype == LLMRS_BF16)
    post_norm_kernel<TY, __nv_bfloat16><<<n_rows, threads, smem, stream>>>(h, (const TY*)y, ls, w,
                                                                          (__nv_bfloat16*)out, width, alpha, eps);
  else
    return llmrs_fail("post_norm: unknown output dtype %d", out_dtype);
  return llmrs_launch_status("post_norm");
}

LLMRS_API int llmrs_post_norm(float* h, const void* y, int y_dtype, const float* ls, const float* w, void* out,
                              int out_dtype, int n_rows, int width, float alpha, float eps, cudaStream_t stream) {
  LLMRS_REQUIRE(n_rows >= 0 && width > 0 && width <= 12288, "post_norm: bad sizes (rows %d, width %d)", n_rows, width);
  if (n_rows == 0) return 0;
  if (y == nullptr || y_dtype == LLMRS_F32)
    return launch_post_norm<float>(h, y, ls, w, out, out_dtype, n_rows, width, alpha, eps, stream);
  if (y_dtype == LLMRS_BF16)
    return launch_post_norm<__nv_bfloat16>(h, y, ls, w, out, out_dtype, n_rows, width, alpha, eps, stream);
  return llmrs_fail("post_norm: unknown dtype %d", y_dtype);
}

template <typename T>
__global__ void relu_sq_kernel(const T* __restrict__ x, T* __restrict__ out, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = fmaxf(to_float(x[i]), 0.f);
  out[i] = from_float<T>(v * v);
}

LLMRS_API int llmrs_relu_sq(const void* x, void* out, long long n, int dtype, cudaStream_t stream) {
  LLMRS_REQUIRE(n >= 0, "relu_sq: bad size");
  if (n == 0) return 0;
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (dtype == LLMRS_F32)
    relu_sq_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, (float*)out, n);
  else if (dtype == LLMRS_BF16)
    relu_sq_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n);
  else
    return llmrs_fail("relu_sq: unknown dtype %d", dtype);
  return llmrs_launch_status("relu_sq");
}

__global__ void scale_kernel(float* __restrict__ z, long long n, float s) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) z[i] *= s;
}

LLMRS_API int llmrs_scale(float* z, long long n, float s, cudaStream_t stream) {
  LLMRS_REQUIRE(n >= 0, "scale: bad size");
  if (n == 0) return 0;
  scale_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(z, n, s);
  return llmrs_launch_status("scale");
}
