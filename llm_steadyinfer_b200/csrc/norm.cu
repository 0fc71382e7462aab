// RMSNorm fused with the residual add that precedes it:
//   h = resid (+ delta);  resid <- h;  out = weight * h * rsqrt(mean(h^2) + eps)
// The reference runs the add (src/source/op/kernels/cuda/add_kernel.cu:4-12) and the
// norm (rmsnorm_kernel.cu:8-60, eps fixed at 1e-6) as separate launches; here eps is an
// argument, the residual stream is fp32, and sum of squares, mean and rsqrt are fp32.
// With `rows` given, output row r is computed from stream row rows[r] and the stream
// is left untouched (used to normalise only the rows whose logits are wanted).
//
// One block per row. When the width is a multiple of 8 every thread moves 8 elements at a
// time with 16-byte loads (all loads of a row are in flight before the first use) and keeps
// them in registers between the two passes; other widths take the scalar kernel, which
// stages the row in shared memory.
#include "common.cuh"

template <typename T> struct Vec8;
template <> struct Vec8<float> {
  float v[8];
  __device__ __forceinline__ void load(const float* p) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  __device__ __forceinline__ void store(float* p) const {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct Vec8<__nv_bfloat16> {
  float v[8];
  __device__ __forceinline__ void load(const __nv_bfloat16* p) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

// CHUNKS: 8-element chunks per thread (hidden <= CHUNKS * 8 * blockDim.x)
template <typename TX, typename TW, int CHUNKS>
__global__ void __launch_bounds__(512) add_rmsnorm_vec_kernel(float* __restrict__ resid, const TX* __restrict__ delta,
                                       const TX* __restrict__ delta2, const int* __restrict__ rows, const TW* __restrict__ weight,
                                       TX* __restrict__ out, int hidden, float eps, int num_rows,
                                       const void* ahead, long long ahead_bytes, int trigger) {
  __shared__ float scratch[33];
  if (trigger) pdl_trigger();
  if ((int)blockIdx.x >= num_rows) {              // blocks behind the rows only fetch ahead
    l2_prefetch_share(ahead, ahead_bytes, blockIdx.x - num_rows, gridDim.x - num_rows);
    return;
  }
  pdl_prologue();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* h = resid + (size_t)src * hidden;
  const TX* dl = delta ? delta + (size_t)src * hidden : nullptr;
  const TX* dl2 = (delta && delta2) ? delta2 + (size_t)src * hidden : nullptr;     // a second result of the same block
  const int nchunks = hidden >> 3;
  Vec8<float> x[CHUNKS];
  Vec8<TX> dv[CHUNKS], dv2[CHUNKS];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunks) {
      x[c].load(h + ch * 8);
      if (dl) dv[c].load(dl + ch * 8);
      if (dl2) dv2[c].load(dl2 + ch * 8);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunks) {
      if (dl) {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[c].v[i] += dv[c].v[i];
        if (dl2) {
#pragma unroll
          for (int i = 0; i < 8; ++i) x[c].v[i] += dv2[c].v[i];
        }
        if (!rows) x[c].store(h + ch * 8);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += x[c].v[i] * x[c].v[i];
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TX* o = out + (size_t)r * hidden;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunks) {
      Vec8<TW> w;
      w.load(weight + ch * 8);
      Vec8<TX> y;
#pragma unroll
      for (int i = 0; i < 8; ++i) y.v[i] = w.v[i] * (x[c].v[i] * inv);
      y.store(o + ch * 8);
    }
  }
}

template <typename TX, typename TW>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TX* __restrict__ delta, const TX* __restrict__ delta2,
                                   const int* __restrict__ rows, const TW* __restrict__ weight,
                                   TX* __restrict__ out, int hidden, float eps) {
  __shared__ float scratch[33];
  extern __shared__ float row_cache[];        // `hidden` floats
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* h = resid + (size_t)src * hidden;
  const TX* dl = delta ? delta + (size_t)src * hidden : nullptr;
  const TX* dl2 = (delta && delta2) ? delta2 + (size_t)src * hidden : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = h[i];
    if (dl) v += to_f32<TX>(dl[i]);
    if (dl2) v += to_f32<TX>(dl2[i]);
    row_cache[i] = v;
    if (dl && !rows) h[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TX* o = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = from_f32<TX>(to_f32<TW>(weight[i]) * (row_cache[i] * inv));
}

template <typename TX, typename TW>
static int launch2(float* resid, const void* delta, const void* delta2, const int* rows, const void* weight, void* out,
                   int num_rows, int hidden, float eps, const void* ahead, long long ahead_bytes, cudaStream_t stream) {
  const TX* d = (const TX*)delta;
  const TX* d2 = (const TX*)delta2;
  const TW* w = (const TW*)weight;
  TX* o = (TX*)out;
  const bool aligned = ((uintptr_t)resid % 16 == 0) && ((uintptr_t)delta % 16 == 0) && ((uintptr_t)delta2 % 16 == 0) &&
                       ((uintptr_t)weight % 16 == 0) && ((uintptr_t)out % 16 == 0);
  if (hidden % 8 == 0 && aligned && hidden <= 4 * 8 * 512) {
    const int nchunks = hidden / 8;
    // threads: a multiple of 32 that covers the row in at most 4 passes
    int threads = nchunks > 256 ? 512 : (nchunks > 128 ? 256 : 128);
    if (num_rows >= 1024 && nchunks <= 1024) threads = min(threads, 256);   // many rows: more blocks per SM
    const int per = (nchunks + threads - 1) / threads;
    // with something to fetch ahead: enough further blocks that every SM takes part
    if (ahead && ahead_bytes < 4096) ahead = nullptr;
    const int trigger = si_pdl_trigger_enabled() && num_rows <= 64;      // a launch of one wave
    const int sms = si_sm_count();
    const int extra = ahead ? max(0, sms - num_rows) + sms : 0;
    const dim3 grid(num_rows + extra);
    if (per <= 1) si_launch(add_rmsnorm_vec_kernel<TX, TW, 1>, grid, dim3(threads), 0, stream, resid, d, d2, rows, w, o, hidden, eps, num_rows, ahead, ahead_bytes, trigger);
    else if (per <= 2) si_launch(add_rmsnorm_vec_kernel<TX, TW, 2>, grid, dim3(threads), 0, stream, resid, d, d2, rows, w, o, hidden, eps, num_rows, ahead, ahead_bytes, trigger);
    else si_launch(add_rmsnorm_vec_kernel<TX, TW, 4>, grid, dim3(threads), 0, stream, resid, d, d2, rows, w, o, hidden, eps, num_rows, ahead, ahead_bytes, trigger);
    return si_last_error();
  }
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return -2;           // hidden too large for the row cache
  auto k = add_rmsnorm_kernel<TX, TW>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  k<<<num_rows, threads, smem, stream>>>(resid, d, d2, rows, w, o, hidden, eps);
  return si_last_error();
}

// x_dtype: dtype of delta, delta2 and out; `delta2` (may be null, and counts only beside `delta`): a second result that
// joins the stream in the same sum, h = (resid + delta) + delta2. `ahead` (may be null): `ahead_bytes` bytes that the kernel after this
// one streams, fetched into L2 meanwhile (a hint: the vectorised kernel takes it, the other one ignores it).
// Returns 0, a CUDA error code, or -2 (size refused).
SI_EXPORT int si_add_rmsnorm(float* resid, const void* delta, const void* delta2, const int* rows, const void* weight,
                             int weight_dtype, void* out, int x_dtype, int num_rows, int hidden,
                             float eps, const void* ahead, long long ahead_bytes, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (x_dtype == SI_BF16) {
    if (weight_dtype == SI_BF16)
      return launch2<__nv_bfloat16, __nv_bfloat16>(resid, delta, delta2, rows, weight, out, num_rows, hidden, eps, ahead, ahead_bytes, stream);
    return launch2<__nv_bfloat16, float>(resid, delta, delta2, rows, weight, out, num_rows, hidden, eps, ahead, ahead_bytes, stream);
  }
  if (weight_dtype == SI_BF16)
    return launch2<float, __nv_bfloat16>(resid, delta, delta2, rows, weight, out, num_rows, hidden, eps, ahead, ahead_bytes, stream);
  return launch2<float, float>(resid, delta, delta2, rows, weight, out, num_rows, hidden, eps, ahead, ahead_bytes, stream);
}

// ---- a norm that is not on the residual stream ------------------------------------------------------------------
// out[r, :] = weight * x[r, :] * rsqrt(mean(x[r, :]^2) + eps) for rows of `n` elements that lie in a two-level
// layout: row r = (a, b) with b < inner starts at x + a * outer_stride + b * inner_stride (the heads of a token
// inside a stacked projection, for a norm over each head; inner = 1 for plain rows). One warp a row, statistics in
// fp32, in place if out == x. Nothing is added and no stream is written: what a mixer calls for a norm of its own.
template <typename TX, typename TW>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const TX* __restrict__ x, TX* __restrict__ out,
                                                           const TW* __restrict__ weight, long long num_rows, int n, int inner,
                                                           long long x_outer, long long x_inner, long long o_outer,
                                                           long long o_inner, float eps) {
  pdl_prologue();
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= num_rows) return;
  const int lane = threadIdx.x & 31;
  const long long a = r / inner, b = r - a * inner;
  const TX* xr = x + a * x_outer + b * x_inner;
  TX* orow = out + a * o_outer + b * o_inner;
  float ss = 0.f;
  for (int i = lane; i < n; i += 32) {
    const float v = to_f32<TX>(xr[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)n + eps);
  for (int i = lane; i < n; i += 32) orow[i] = from_f32<TX>(to_f32<TW>(weight[i]) * (to_f32<TX>(xr[i]) * inv));
}

template <typename TX, typename TW>
static int rows_launch(const void* x, void* out, const void* weight, long long num_rows, int n, int inner, long long x_outer,
                       long long x_inner, long long o_outer, long long o_inner, float eps, cudaStream_t stream) {
  const long long blocks = (num_rows + 7) / 8;
  if (blocks > 0x7fffffffLL) return -2;
  si_launch(rmsnorm_rows_kernel<TX, TW>, dim3((unsigned)blocks), dim3(256), 0, stream, (const TX*)x, (TX*)out, (const TW*)weight,
            num_rows, n, inner, x_outer, x_inner, o_outer, o_inner, eps);
  return si_last_error();
}

// x_dtype: dtype of x and out; strides in elements. Returns 0, a CUDA error code, or -2 (size refused).
SI_EXPORT int si_rmsnorm_rows(const void* x, void* out, int x_dtype, const void* weight, int weight_dtype, long long num_rows,
                              int n, int inner, long long x_outer, long long x_inner, long long o_outer, long long o_inner,
                              float eps, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (n <= 0 || inner <= 0) return -2;
  if (x_dtype == SI_BF16) {
    if (weight_dtype == SI_BF16)
      return rows_launch<__nv_bfloat16, __nv_bfloat16>(x, out, weight, num_rows, n, inner, x_outer, x_inner, o_outer, o_inner, eps, stream);
    return rows_launch<__nv_bfloat16, float>(x, out, weight, num_rows, n, inner, x_outer, x_inner, o_outer, o_inner, eps, stream);
  }
  if (weight_dtype == SI_BF16) return -2;
  return rows_launch<float, float>(x, out, weight, num_rows, n, inner, x_outer, x_inner, o_outer, o_inner, eps, stream);
}


// ---- the add in its general form --------------------------------------------------------------------------------
// What blocks with a norm behind each sublayer, and models that feed something into the stream between layers, need:
//   d  = delta (+ delta_bias)                                    the sublayer's result
//   d' = delta_weight * d * rsqrt(mean(d^2) + delta_eps)         when delta_weight is given, else d' = d
//   h  = resid + d' (+ extra[row]) (+ vec);   resid <- h  (not with `rows`)
//   out = weight * h * rsqrt(mean(h^2) + eps)                    when out is given
// delta, extra, vec, out may each be absent. All statistics and sums are fp32. One block a row; the row (and the
// delta's) is staged in shared memory, so any width up to what shared memory holds.
template <typename TX, typename TW>
__global__ void __launch_bounds__(256) add_norm_general_kernel(float* __restrict__ resid, const TX* __restrict__ delta,
    const float* __restrict__ delta_bias, const TW* __restrict__ delta_weight, float delta_eps,
    const float* __restrict__ extra, const float* __restrict__ vec, const int* __restrict__ rows,
    const TW* __restrict__ weight, TX* __restrict__ out, int hidden, float eps) {
  __shared__ float scratch[33];
  extern __shared__ float row_cache[];        // `hidden` floats
  pdl_prologue();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* h = resid + (size_t)src * hidden;
  float dscale = 1.f;
  if (delta && delta_weight) {
    const TX* dl = delta + (size_t)src * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float v = to_f32<TX>(dl[i]) + (delta_bias ? delta_bias[i] : 0.f);
      ss += v * v;
    }
    ss = block_sum(ss, scratch);
    dscale = rsqrtf(ss / (float)hidden + delta_eps);
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = h[i];
    if (delta) {
      float d = to_f32<TX>(delta[(size_t)src * hidden + i]) + (delta_bias ? delta_bias[i] : 0.f);
      if (delta_weight) d = to_f32<TW>(delta_weight[i]) * (d * dscale);
      v += d;
    }
    if (extra) v += extra[(size_t)src * hidden + i];
    if (vec) v += vec[i];
    row_cache[i] = v;
    if (!rows) h[i] = v;
    ss += v * v;
  }
  if (!out) return;
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TX* o = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = from_f32<TX>(to_f32<TW>(weight[i]) * (row_cache[i] * inv));
}

// The same with the row in registers: widths that are multiples of 8 with 16-byte aligned tensors; every thread moves
// 8 elements at a time with 16-byte loads, all of a row's loads in flight before the first use.
template <typename TX, typename TW, int CHUNKS>
__global__ void __launch_bounds__(512) add_norm_general_vec_kernel(float* __restrict__ resid, const TX* __restrict__ delta,
    const float* __restrict__ delta_bias, const TW* __restrict__ delta_weight, float delta_eps,
    const float* __restrict__ extra, const float* __restrict__ vec, const int* __restrict__ rows,
    const TW* __restrict__ weight, TX* __restrict__ out, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_prologue();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* h = resid + (size_t)src * hidden;
  const int nchunks = hidden >> 3;
  Vec8<float> x[CHUNKS], d[CHUNKS];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunks) {
      x[c].load(h + ch * 8);
      if (delta) {
        Vec8<TX> t;
        t.load(delta + (size_t)src * hidden + ch * 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) d[c].v[i] = t.v[i];
        if (delta_bias) {
          Vec8<float> b;
          b.load(delta_bias + ch * 8);
#pragma unroll
          for (int i = 0; i < 8; ++i) d[c].v[i] += b.v[i];
        }
      }
    }
  }
  if (delta && delta_weight) {
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
      if (threadIdx.x + c * blockDim.x < nchunks)
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += d[c].v[i] * d[c].v[i];
    ss = block_sum(ss, scratch);
    const float dscale = rsqrtf(ss / (float)hidden + delta_eps);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
      if (ch < nchunks) {
        Vec8<TW> w;
        w.load(delta_weight + ch * 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) d[c].v[i] = w.v[i] * (d[c].v[i] * dscale);
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunks) {
      if (delta)
#pragma unroll
        for (int i = 0; i < 8; ++i) x[c].v[i] += d[c].v[i];
      if (extra) {
        Vec8<float> e;
        e.load(extra + (size_t)src * hidden + ch * 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[c].v[i] += e.v[i];
      }
      if (vec) {
        Vec8<float> e;
        e.load(vec + ch * 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[c].v[i] += e.v[i];
      }
      if (!rows) x[c].store(h + ch * 8);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += x[c].v[i] * x[c].v[i];
    }
  }
  if (!out) return;
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TX* o = out + (size_t)r * hidden;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunks) {
      Vec8<TW> w;
      w.load(weight + ch * 8);
      Vec8<TX> yv;
#pragma unroll
      for (int i = 0; i < 8; ++i) yv.v[i] = w.v[i] * (x[c].v[i] * inv);
      yv.store(o + ch * 8);
    }
  }
}

template <typename TX, typename TW>
static int general_launch(float* resid, const void* delta, const float* delta_bias, const void* delta_weight, float delta_eps,
                          const float* extra, const float* vec, const int* rows, const void* weight, void* out, int num_rows,
                          int hidden, float eps, cudaStream_t stream) {
  const auto al = [](const void* p) { return ((uintptr_t)p % 16) == 0; };
  if (hidden % 8 == 0 && hidden <= 4 * 8 * 512 && al(resid) && al(delta) && al(delta_bias) && al(delta_weight) && al(extra) &&
      al(vec) && al(weight) && al(out)) {
    const int nchunks = hidden / 8;
    int threads = nchunks > 256 ? 512 : (nchunks > 128 ? 256 : 128);
    if (num_rows >= 1024 && nchunks <= 1024) threads = min(threads, 256);   // many rows: more blocks per SM
    const int per = (nchunks + threads - 1) / threads;
#define SI_GENERAL_VEC(C)                                                                                             \
    si_launch(add_norm_general_vec_kernel<TX, TW, C>, dim3(num_rows), dim3(threads), 0, stream, resid, (const TX*)delta,   \
              delta_bias, (const TW*)delta_weight, delta_eps, extra, vec, rows, (const TW*)weight, (TX*)out, hidden, eps)
    if (per <= 1) SI_GENERAL_VEC(1);
    else if (per <= 2) SI_GENERAL_VEC(2);
    else SI_GENERAL_VEC(4);
#undef SI_GENERAL_VEC
    return si_last_error();
  }
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return -2;
  static size_t configured = 0;
  auto k = add_norm_general_kernel<TX, TW>;
  if (smem > 48 * 1024 && smem > configured) {
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -2;
    configured = smem;
  }
  si_launch(k, dim3(num_rows), dim3(hidden >= 1024 ? 256 : 128), smem, stream, resid, (const TX*)delta, delta_bias,
            (const TW*)delta_weight, delta_eps, extra, vec, rows, (const TW*)weight, (TX*)out, hidden, eps);
  return si_last_error();
}

// x_dtype: dtype of delta and out; weight_dtype: dtype of weight and delta_weight. Returns 0, a CUDA error code, or -2.
SI_EXPORT int si_add_norm_general(float* resid, const void* delta, const float* delta_bias, const void* delta_weight,
                                  float delta_eps, const float* extra, const float* vec, const int* rows,
                                  const void* weight, int weight_dtype, void* out, int x_dtype, int num_rows, int hidden,
                                  float eps, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (out && !weight) return -2;
  if (x_dtype == SI_BF16) {
    if (weight_dtype == SI_BF16)
      return general_launch<__nv_bfloat16, __nv_bfloat16>(resid, delta, delta_bias, delta_weight, delta_eps, extra, vec, rows, weight, out, num_rows, hidden, eps, stream);
    return general_launch<__nv_bfloat16, float>(resid, delta, delta_bias, delta_weight, delta_eps, extra, vec, rows, weight, out, num_rows, hidden, eps, stream);
  }
  if (weight_dtype == SI_BF16)
    return general_launch<float, __nv_bfloat16>(resid, delta, delta_bias, delta_weight, delta_eps, extra, vec, rows, weight, out, num_rows, hidden, eps, stream);
  return general_launch<float, float>(resid, delta, delta_bias, delta_weight, delta_eps, extra, vec, rows, weight, out, num_rows, hidden, eps, stream);
}

// ---- sublayer results through learned gates into the stream ---------------------------------------------------------------
//   resid[t, :] += mult * (sigmoid(z1[t, :] + b1) * a[t, :] + sigmoid(z2[t, :] + b2) * f[t, :])
// for blocks whose sublayers read the same stream side by side and are each gated, entry by entry, by a projection of
// their own input (the second pair absent: one sublayer). z, a, f in the compute dtype, b fp32 [d], sums in fp32.
template <typename T>
__global__ void __launch_bounds__(256) gated_add_kernel(float* __restrict__ resid, const T* __restrict__ z1, const float* __restrict__ b1,
    const T* __restrict__ a, const T* __restrict__ z2, const float* __restrict__ b2, const T* __restrict__ f, long long n, int d,
    float mult) {
  pdl_prologue();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % d);
    float s = to_f32<T>(a[idx]) / (1.f + expf(-(to_f32<T>(z1[idx]) + b1[c])));
    if (z2) s += to_f32<T>(f[idx]) / (1.f + expf(-(to_f32<T>(z2[idx]) + b2[c])));
    resid[idx] = fmaf(mult, s, resid[idx]);
  }
}

// The same, eight entries a thread with 16-byte loads (d a multiple of 8, every tensor 16-byte aligned).
template <typename T>
__global__ void __launch_bounds__(256) gated_add_vec_kernel(float* __restrict__ resid, const T* __restrict__ z1,
    const float* __restrict__ b1, const T* __restrict__ a, const T* __restrict__ z2, const float* __restrict__ b2,
    const T* __restrict__ f, long long n8, int d8, float mult) {
  pdl_prologue();
  for (long long i8 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i8 < n8; i8 += (long long)gridDim.x * blockDim.x) {
    const long long idx = i8 * 8;
    const int c = (int)(i8 % d8) * 8;
    Vec8<T> vz, va;
    Vec8<float> vr, vb;
    vz.load(z1 + idx); va.load(a + idx); vr.load(resid + idx); vb.load(b1 + c);
    float s[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) s[e] = va.v[e] / (1.f + expf(-(vz.v[e] + vb.v[e])));
    if (z2) {
      vz.load(z2 + idx); va.load(f + idx); vb.load(b2 + c);
#pragma unroll
      for (int e = 0; e < 8; ++e) s[e] += va.v[e] / (1.f + expf(-(vz.v[e] + vb.v[e])));
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) vr.v[e] = fmaf(mult, s[e], vr.v[e]);
    vr.store(resid + idx);
  }
}

SI_EXPORT int si_gated_add(float* resid, const void* z1, const float* b1, const void* a, const void* z2, const float* b2,
                           const void* f, int dtype, int rows, int d, float mult, cudaStream_t stream) {
  if (rows <= 0 || d <= 0) return 0;
  if (!z1 || !b1 || !a || ((z2 != nullptr) != (f != nullptr)) || (z2 && !b2)) return -2;
  const long long n = (long long)rows * d;
  const int threads = 256;
  const uintptr_t all = (uintptr_t)resid | (uintptr_t)z1 | (uintptr_t)b1 | (uintptr_t)a | (uintptr_t)z2 | (uintptr_t)b2 | (uintptr_t)f;
  if (d % 8 == 0 && (all & 15) == 0) {
    const long long n8 = n / 8, want8 = (n8 + threads - 1) / threads;
    const int blocks8 = (int)(want8 < 8LL * si_sm_count() ? want8 : 8LL * si_sm_count());
    if (dtype == SI_BF16)
      si_launch(gated_add_vec_kernel<__nv_bfloat16>, dim3(blocks8), dim3(threads), 0, stream, resid, (const __nv_bfloat16*)z1, b1,
                (const __nv_bfloat16*)a, (const __nv_bfloat16*)z2, b2, (const __nv_bfloat16*)f, n8, d / 8, mult);
    else
      si_launch(gated_add_vec_kernel<float>, dim3(blocks8), dim3(threads), 0, stream, resid, (const float*)z1, b1, (const float*)a,
                (const float*)z2, b2, (const float*)f, n8, d / 8, mult);
    return si_last_error();
  }
  const long long want = (n + threads - 1) / threads;
  const int blocks = (int)(want < 8LL * si_sm_count() ? want : 8LL * si_sm_count());
  if (dtype == SI_BF16)
    si_launch(gated_add_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, resid, (const __nv_bfloat16*)z1, b1,
              (const __nv_bfloat16*)a, (const __nv_bfloat16*)z2, b2, (const __nv_bfloat16*)f, n, d, mult);
  else
    si_launch(gated_add_kernel<float>, dim3(blocks), dim3(threads), 0, stream, resid, (const float*)z1, b1, (const float*)a,
              (const float*)z2, b2, (const float*)f, n, d, mult);
  return si_last_error();
}
