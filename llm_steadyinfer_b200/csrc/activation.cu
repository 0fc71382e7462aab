// Elementwise activations of feed-forwards without a gate: out[t, f] = act(in[t, f]), fp32 arithmetic.
//   0 relu(x)^2     1 gelu_tanh(x) = 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))     2 silu(x)     3 relu(x)
#include "common.cuh"
#include <math.h>

__device__ __forceinline__ float act_apply(float x, int kind) {
  switch (kind) {
    case 0: { const float r = fmaxf(x, 0.f); return r * r; }
    case 1: return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    case 2: return x / (1.f + expf(-x));
    default: return fmaxf(x, 0.f);
  }
}

template <typename T>
__global__ void activation_kernel(const T* __restrict__ in, long long in_stride, T* __restrict__ out,
                                  long long out_stride, int rows, int width, int kind) {
  pdl_prologue();
  const long long n = (long long)rows * width;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / width, f = idx % width;
    out[t * out_stride + f] = from_f32<T>(act_apply(to_f32<T>(in[t * in_stride + f]), kind));
  }
}

SI_EXPORT int si_activation(const void* in, long long in_stride, void* out, long long out_stride, int dtype, int rows,
                            int width, int kind, cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  if (kind < 0 || kind > 3) return -2;
  const long long n = (long long)rows * width;
  const int threads = 256;
  const long long want = (n + threads - 1) / threads;
  const int blocks = (int)(want < 8LL * si_sm_count() ? want : 8LL * si_sm_count());
  if (dtype == SI_BF16)
    si_launch(activation_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)in, in_stride,
              (__nv_bfloat16*)out, out_stride, rows, width, kind);
  else
    si_launch(activation_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)in, in_stride, (float*)out,
              out_stride, rows, width, kind);
  return si_last_error();
}

// x <- cap * tanh(x / cap) in place on fp32 values (a soft limit on logits).
__global__ void softcap_kernel(float* __restrict__ x, long long n, float cap) {
  pdl_prologue();
  const float inv = 1.f / cap;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x)
    x[idx] = cap * tanhf(x[idx] * inv);
}

SI_EXPORT int si_softcap(float* x, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!(cap > 0.f)) return -2;
  const int threads = 256;
  const long long want = (n + threads - 1) / threads;
  const int blocks = (int)(want < 8LL * si_sm_count() ? want : 8LL * si_sm_count());
  si_launch(softcap_kernel, dim3(blocks), dim3(threads), 0, stream, x, n, cap);
  return si_last_error();
}

// x[t, f] += bias[f] (fp32 sum, stored in x's dtype): the bias of a product whose kernel has no epilogue for it.
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, long long stride, const float* __restrict__ bias, int rows, int width) {
  pdl_prologue();
  const long long n = (long long)rows * width;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / width, f = idx % width;
    x[t * stride + f] = from_f32<T>(to_f32<T>(x[t * stride + f]) + bias[f]);
  }
}

SI_EXPORT int si_add_bias(void* x, long long stride, int dtype, const float* bias, int rows, int width, cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  const long long n = (long long)rows * width;
  const int threads = 256;
  const long long want = (n + threads - 1) / threads;
  const int blocks = (int)(want < 8LL * si_sm_count() ? want : 8LL * si_sm_count());
  if (dtype == SI_BF16)
    si_launch(add_bias_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (__nv_bfloat16*)x, stride, bias, rows, width);
  else
    si_launch(add_bias_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (float*)x, stride, bias, rows, width);
  return si_last_error();
}
