// The gated delta rule: a linear-attention recurrence whose state is a matrix per head that forgets by a scalar
// decay and is corrected, not just added to, by each token:
//   S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t          S is dk x dv, fp32
// so the read-out sees the token's own write. Everything that enters the recurrence is fp32.
//
// Two kernels. `delta_prepare` works on all rows at once: it makes q and k unit vectors per head
// (x / sqrt(sum(x^2) + 1e-6), q also times `q_scale`), beta = sigmoid(b), g = exp(-exp(A_log) * softplus(a + dt_bias))
// and q . k of the prepared vectors.
// `delta_scan` walks the tokens of every sequence of the step in order. The columns of S are independent of one
// another, so a block takes (sequence, head, a cut of the columns); thread (column j, part p) keeps RPT neighbouring
// rows of column j in registers. Per token it forms its parts of k . S[:, j] and q . S[:, j] from the old state (two
// rows at a time on the packed fp32 instructions, two sums each, so that the chain of dependent additions is short),
// the NP parts of a column (neighbouring lanes) are added with shuffles, and then
//   kS = g (k . S_old[:, j]);  u_j = beta (v_j - kS);  o_j = g (q . S_old[:, j]) + (q . k) u_j;  S[:, j] <- g S_old[:, j] + k u_j
// which is the order above with one pass over the registers for the sums and one for the update. q, k, v, beta, g and
// q . k of CHUNK tokens arrive by cp.async in the half of shared memory that is not being computed on; within a chunk
// the warps do not wait for one another.
// A request's state lies at the start of its slot, head by head, each head as [RPT][dv][NP] (see delta_shape); a
// portion that begins at position 0 starts from zero whatever the slot held.
#include "common.cuh"
#include <math.h>

__device__ __forceinline__ float softplus_d(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// xc: fp32 rows [q: G*dk | k: G*dk | ...] (the convolution's output), normalised in place.
// ba: rows of the projection holding b (H values at b_off) and a (H values at a_off) in the compute dtype.
// bg: fp32 [T, 2H + G]: beta, then g, then q . k of the prepared vectors per query/key head.
template <typename T>
__global__ void __launch_bounds__(128) delta_prepare_kernel(float* __restrict__ xc, long long xc_stride, const T* __restrict__ ba,
    long long ba_stride, int b_off, int a_off, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
    float* __restrict__ bg, int G, int H, int dk, float q_scale) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float* row = xc + (size_t)t * xc_stride;
  float* bgr = bg + (size_t)t * (2 * H + G);
  for (int gh = warp; gh < G; gh += nwarps) {          // a warp takes the query and the key of one head
    float* q = row + (size_t)gh * dk;
    float* k = row + (size_t)(G + gh) * dk;
    float sq = 0.f, sk = 0.f;
    for (int i = lane; i < dk; i += 32) { sq += q[i] * q[i]; sk += k[i] * k[i]; }
    const float fq = rsqrtf(warp_sum(sq) + 1e-6f) * q_scale, fk = rsqrtf(warp_sum(sk) + 1e-6f);
    float dot = 0.f;
    for (int i = lane; i < dk; i += 32) {
      const float a = q[i] * fq, b = k[i] * fk;
      q[i] = a; k[i] = b;
      dot = fmaf(a, b, dot);
    }
    dot = warp_sum(dot);
    if (lane == 0) bgr[2 * H + gh] = dot;
  }
  const T* r = ba + (size_t)t * ba_stride;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    bgr[h] = 1.f / (1.f + expf(-to_f32<T>(r[b_off + h])));
    bgr[H + h] = expf(-expf(a_log[h]) * softplus_d(to_f32<T>(r[a_off + h]) + dt_bias[h]));
  }
}

SI_EXPORT int si_delta_prepare(float* xc, long long xc_stride, const void* ba, int dtype, long long ba_stride, int b_off,
                               int a_off, const float* a_log, const float* dt_bias, float* bg, int num_tokens, int G, int H,
                               int dk, float q_scale, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (dtype == SI_BF16)
    si_launch(delta_prepare_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), 0, stream, xc, xc_stride,
              (const __nv_bfloat16*)ba, ba_stride, b_off, a_off, a_log, dt_bias, bg, G, H, dk, q_scale);
  else
    si_launch(delta_prepare_kernel<float>, dim3(num_tokens), dim3(128), 0, stream, xc, xc_stride, (const float*)ba,
              ba_stride, b_off, a_off, a_log, dt_bias, bg, G, H, dk, q_scale);
  return si_last_error();
}

#define DELTA_CHUNK 32

__device__ __forceinline__ void delta_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void delta_cp16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}

// The shape for a state of dk x dv: rows a thread (RPT, a multiple of 4) and parts a column (NP, a power of two up to 32,
// RPT * NP >= dk): about sixteen parts. A sequence's tokens are a chain of dependent steps; few rows a thread shorten the
// chain and give a multiprocessor warps to choose from, many parts cost shuffles (measured at 128 x 128, 16 heads, one
// sequence of 2,048 tokens: 16 rows in 8 parts 1.54 ms, 4 rows in 32 parts 0.69 ms).
// Thread (column j, part p) keeps, for c < RPT / 4, the four rows (c * NP + p) * 4 .. + 3 of column j (so that the parts
// read neighbouring 16-byte words of q and k). A head's state lies in the slot as [RPT][dv][NP]: entry
// ((r * dv + j) * NP + p) is the thread's r-th row, so that a block reads and writes whole lines whatever cut of the
// columns it has.
struct DeltaShape { int rpt, np; };
static DeltaShape delta_shape(int dk) {
  DeltaShape s;
  s.rpt = ((dk + 15) / 16 + 3) / 4 * 4;
  int parts = 1;
  while (parts * s.rpt < dk) parts *= 2;
  s.np = parts;
  return s;
}
// fp32 entries of one head's state in a slot
SI_EXPORT long long si_delta_state_floats(int dk, int dv) {
  if (dk <= 0 || dv <= 0 || dk > 512) return -1;
  const DeltaShape s = delta_shape(dk);
  return (long long)s.rpt * s.np * dv;
}

// RPT: rows of a column that a thread keeps, as RPT / 2 pairs (the sums and the update run two rows at a time on the
// packed fp32 instructions). Shared memory: two buffers of CHUNK tokens of [q: RPT * NP | k: RPT * NP | v: cols |
// beta, g, q . k, -] (rows beyond dk stay zero), filled by cp.async one chunk ahead of the sums.
template <int RPT, int NP>
__global__ void __launch_bounds__(256) delta_scan_kernel(const float* __restrict__ xc, long long xc_stride,
    const float* __restrict__ bg, int bg_width, float* __restrict__ state, long long state_stride, float* __restrict__ y,
    long long y_stride, const int* __restrict__ q_start, const int* __restrict__ ctx_len, const int* __restrict__ slots,
    int G, int H, int dk, int dv, int cols) {
  extern __shared__ __align__(16) float sm[];
  pdl_prologue();
  const int s = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * cols;
  const int row0 = q_start[s], n = q_start[s + 1] - row0;
  if (n <= 0) return;
  const int pos0 = ctx_len[s] - n;
  const int g = h / (H / G);
  const int p = threadIdx.x % NP, jl = threadIdx.x / NP;
  const int j = j0 + jl;
  const bool col_ok = jl < cols && j < dv;
  float* S = state + (size_t)slots[s] * state_stride + (size_t)h * RPT * NP * dv + (size_t)(col_ok ? j : 0) * NP + p;
  const size_t s_step = (size_t)dv * NP;
  float2 st[RPT / 2];
#pragma unroll
  for (int r = 0; r < RPT / 2; ++r) {
    st[r].x = (col_ok && pos0 > 0) ? S[(size_t)(2 * r) * s_step] : 0.f;
    st[r].y = (col_ok && pos0 > 0) ? S[(size_t)(2 * r + 1) * s_step] : 0.f;
  }
  const int dkp = RPT * NP;
  const int per_tok = 2 * dkp + ((cols + 3) & ~3) + 4;
  for (int idx = threadIdx.x; idx < 2 * DELTA_CHUNK * per_tok; idx += blockDim.x) sm[idx] = 0.f;
  __syncthreads();
  const size_t q_off = (size_t)g * dk, k_off = (size_t)(G + g) * dk, v_off = (size_t)2 * G * dk + (size_t)h * dv + j0;
  const bool wide = dk % 4 == 0 && xc_stride % 4 == 0 && ((uintptr_t)xc & 15) == 0;      // q and k rows in 16-byte pieces
  // a warp fetches whole tokens (every nwarps-th of the chunk): the copies' bookkeeping is then paid once a token by one
  // warp, not by every warp
  const int unit = wide ? 4 : 1, pieces = 2 * dk / unit, per_half = dk / unit;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  auto fetch = [&](int c0, int buf) {
    const int cn = min(DELTA_CHUNK, n - c0);
    for (int tt = warp; tt < cn; tt += nwarps) {
      float* dst = sm + ((size_t)buf * DELTA_CHUNK + tt) * per_tok;
      const float* row = xc + (size_t)(row0 + c0 + tt) * xc_stride;
      const float* bgr = bg + (size_t)(row0 + c0 + tt) * bg_width;
      for (int t = lane; t < pieces; t += 32) {
        const bool is_q = t < per_half;
        const int i = (is_q ? t : t - per_half) * unit;
        if (wide) delta_cp16(dst + (is_q ? 0 : dkp) + i, row + (is_q ? q_off : k_off) + i);
        else delta_cp4(dst + (is_q ? 0 : dkp) + i, row + (is_q ? q_off : k_off) + i);
      }
      for (int e = lane; e < cols + 3; e += 32) {
        if (e < cols) {
          if (j0 + e < dv) delta_cp4(dst + 2 * dkp + e, row + v_off + e);
        } else {                                     // beta, g, q . k of this head
          const int w = e - cols;
          delta_cp4(dst + per_tok - 4 + w, bgr + (w == 0 ? h : w == 1 ? H + h : 2 * H + g));
        }
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  fetch(0, 0);
  int buf = 0;
  for (int c0 = 0; c0 < n; c0 += DELTA_CHUNK, buf ^= 1) {
    const int cn = min(DELTA_CHUNK, n - c0);
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();                            // this chunk has arrived, and everyone is done with the other buffer
    if (c0 + DELTA_CHUNK < n) fetch(c0 + DELTA_CHUNK, buf ^ 1);
    const float* tok = sm + (size_t)buf * DELTA_CHUNK * per_tok;
    float* yp = y + (size_t)(row0 + c0) * y_stride + (size_t)h * dv + j;
#pragma unroll 2
    for (int tt = 0; tt < cn; ++tt, tok += per_tok, yp += y_stride) {
      const float4* q4 = reinterpret_cast<const float4*>(tok) + p;
      const float4* k4 = reinterpret_cast<const float4*>(tok + dkp) + p;
      float2 kk[RPT / 2];
      float2 sk0 = make_float2(0.f, 0.f), sq0 = sk0;
#pragma unroll
      for (int c = 0; c < RPT / 4; ++c) {
        const float4 kv = k4[c * NP], qv = q4[c * NP];
        kk[2 * c] = make_float2(kv.x, kv.y);
        kk[2 * c + 1] = make_float2(kv.z, kv.w);
        sk0 = __ffma2_rn(kk[2 * c], st[2 * c], sk0);
        sq0 = __ffma2_rn(make_float2(qv.x, qv.y), st[2 * c], sq0);
        sk0 = __ffma2_rn(kk[2 * c + 1], st[2 * c + 1], sk0);
        sq0 = __ffma2_rn(make_float2(qv.z, qv.w), st[2 * c + 1], sq0);
      }
      float sk = sk0.x + sk0.y, sq = sq0.x + sq0.y;
#pragma unroll
      for (int o = 1; o < NP; o <<= 1) {
        sk += __shfl_xor_sync(0xffffffffu, sk, o);
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
      }
      const float4 sc = *reinterpret_cast<const float4*>(tok + per_tok - 4);      // beta, g, q . k
      const float vj = col_ok ? tok[2 * dkp + jl] : 0.f;
      const float u = sc.x * (vj - sc.y * sk);
      const float2 u2 = make_float2(u, u), g2 = make_float2(sc.y, sc.y);
#pragma unroll
      for (int r = 0; r < RPT / 2; ++r) st[r] = __ffma2_rn(kk[r], u2, __fmul2_rn(g2, st[r]));
      if (p == 0 && col_ok) *yp = fmaf(sc.z, u, sc.y * sq);
    }
  }
  if (col_ok) {
#pragma unroll
    for (int r = 0; r < RPT / 2; ++r) {
      S[(size_t)(2 * r) * s_step] = st[r].x;
      S[(size_t)(2 * r + 1) * s_step] = st[r].y;
    }
  }
}

SI_EXPORT int si_delta_scan(const float* xc, long long xc_stride, const float* bg, int bg_width, float* state,
                            long long state_stride, float* y, long long y_stride, const int* q_start, const int* ctx_len,
                            const int* slots, int num_seqs, int G, int H, int dk, int dv, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (G <= 0 || H % G || dk <= 0 || dv <= 0 || dk > 512 || H > 65535 || bg_width < 2 * H + G) return -2;
  const DeltaShape sh = delta_shape(dk);
  if (sh.rpt * sh.np < dk) return -2;
  if (state_stride < (long long)H * sh.rpt * sh.np * dv) return -2;
  // columns a block: as many as 256 threads hold, fewer while the blocks do not fill the device (a block's tokens are a
  // chain of dependent steps, so more blocks of fewer columns finish sooner); never less than a warp
  int cols = 256 / sh.np;
  if (cols > dv) cols = dv;
  if (cols < 1) cols = 1;
  const long long per = (long long)num_seqs * H;
  while (cols > 1 && (cols / 2) * sh.np >= 32 && per * ((dv + cols - 1) / cols) < si_sm_count()) cols /= 2;
  const int zb = (dv + cols - 1) / cols;
  if (zb > 65535) return -2;
  const int threads = ((cols * sh.np + 31) / 32) * 32;
  const size_t smem = (size_t)2 * DELTA_CHUNK * (2 * sh.np * sh.rpt + ((cols + 3) & ~3) + 4) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  const dim3 grid(num_seqs, H, zb), block(threads);
#define DELTA_LAUNCH(R, P)                                                                                           \
  {                                                                                                                  \
    static size_t configured = 0;                                                                                    \
    if (smem > 48 * 1024 && smem > configured) {                                                                     \
      if (cudaFuncSetAttribute(delta_scan_kernel<R, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
        return -2;                                                                                                   \
      configured = smem;                                                                                             \
    }                                                                                                                \
    si_launch(delta_scan_kernel<R, P>, grid, block, smem, stream, xc, xc_stride, bg, bg_width, state, state_stride, y, \
              y_stride, q_start, ctx_len, slots, G, H, dk, dv, cols);                                                \
  }
  // (rows a thread, parts a column) as delta_shape gives them: four rows in 1 to 16 parts up to dk = 64, then 16 parts
  if (sh.np < 16) {
    if (sh.rpt != 4) return -2;
    switch (sh.np) {
      case 1: DELTA_LAUNCH(4, 1) break;
      case 2: DELTA_LAUNCH(4, 2) break;
      case 4: DELTA_LAUNCH(4, 4) break;
      case 8: DELTA_LAUNCH(4, 8) break;
      default: return -2;
    }
  } else if (sh.np == 16) {
    switch (sh.rpt) {                        // dk up to 512: up to 32 rows a thread
      case 4: DELTA_LAUNCH(4, 16) break;
      case 8: DELTA_LAUNCH(8, 16) break;
      case 12: DELTA_LAUNCH(12, 16) break;
      case 16: DELTA_LAUNCH(16, 16) break;
      case 20: DELTA_LAUNCH(20, 16) break;
      case 24: DELTA_LAUNCH(24, 16) break;
      case 28: DELTA_LAUNCH(28, 16) break;
      case 32: DELTA_LAUNCH(32, 16) break;
      default: return -2;
    }
  } else {
    return -2;
  }
#undef DELTA_LAUNCH
  return si_last_error();
}

// ---- the read-out's norm and gate ------------------------------------------------------------------------------------
//   out[t, h, :] = post * w_h * o[t, h, :] * rsqrt(mean(o[t, h, :]^2) + eps) * silu(z[t, h, :])
// w [dv] shared by the heads (w_head_stride 0) or [H, dv] with one row a head (w_head_stride dv); post one number.
// o fp32, z and out in the compute dtype (z and out views with a row stride). One warp a (row, head).
template <typename T>
__global__ void __launch_bounds__(256) head_norm_gate_kernel(const float* __restrict__ o, long long o_stride, const T* __restrict__ z,
    long long z_stride, const float* __restrict__ w, T* __restrict__ out, long long out_stride, long long pairs, int H, int dv,
    float eps, long long w_head_stride, float post) {
  pdl_prologue();
  const long long wi = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wi >= pairs) return;
  const int lane = threadIdx.x & 31;
  const long long t = wi / H;
  const int h = (int)(wi - t * H);
  const float* orow = o + t * o_stride + (size_t)h * dv;
  const T* zr = z + t * z_stride + (size_t)h * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss += orow[i] * orow[i];
  const float rs = rsqrtf(warp_sum(ss) / (float)dv + eps) * post;
  w += (size_t)h * w_head_stride;
  T* dst = out + t * out_stride + (size_t)h * dv;
  for (int i = lane; i < dv; i += 32) {
    const float zz = to_f32<T>(zr[i]);
    dst[i] = from_f32<T>(orow[i] * rs * w[i] * (zz / (1.f + expf(-zz))));
  }
}

SI_EXPORT int si_head_norm_gate(const float* o, long long o_stride, const void* z, int dtype, long long z_stride,
                                const float* w, void* out, long long out_stride, int rows, int H, int dv, float eps,
                                long long w_head_stride, float post, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || dv <= 0) return -2;
  const long long pairs = (long long)rows * H;
  const dim3 grid((unsigned)((pairs + 7) / 8)), block(256);
  if (dtype == SI_BF16)
    si_launch(head_norm_gate_kernel<__nv_bfloat16>, grid, block, 0, stream, o, o_stride, (const __nv_bfloat16*)z, z_stride, w,
              (__nv_bfloat16*)out, out_stride, pairs, H, dv, eps, w_head_stride, post);
  else
    si_launch(head_norm_gate_kernel<float>, grid, block, 0, stream, o, o_stride, (const float*)z, z_stride, w, (float*)out,
              out_stride, pairs, H, dv, eps, w_head_stride, post);
  return si_last_error();
}
