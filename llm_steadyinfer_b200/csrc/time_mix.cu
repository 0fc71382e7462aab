// Time mixing with a decaying matrix state (the recurrence of RWKV-style mixers): per head a state S of n x n that
// forgets by a decay per key channel and gains each token's outer product, read with a bonus for the current token:
//   o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t;      S_t = diag(w_t) S_(t-1) + k_t v_t^T          S fp32, zero at the start
// Three kernels.
// `shift_mix`: the inputs of the mixer's products. Each product s reads x_t + (x_(t-1) - x_t) * mu_s, where x_(t-1) is
// the row before in the same sequence: the step's own row, or for a portion's first row what the slot keeps from the
// step before (zeros at position 0). The blocks of a portion's first row also renew the slot with the portion's last
// row, each its own share of the entries, so no two blocks touch an entry of a slot.
// `time_mix_prepare`: decay = exp(-exp(W2 tanh(z) + w0)) per row and channel (z the low-rank product's first half, fp32
// arithmetic throughout), written beside fp32 copies of r, k, v as rows [r | k | v | decay].
// `decay_scan`: the recurrence. The columns of S are independent, so a block takes (sequence, head, a cut of the
// columns); thread (column j, part p) keeps RPT neighbouring rows of column j in registers, the NP parts of a column are
// neighbouring lanes whose partial read-outs are added with shuffles. r, k, decay and v of CHUNK tokens arrive by
// cp.async in the half of shared memory that is not being computed on. A head's state lies in the slot as
// [RPT][n][NP] (entry ((r * n + j) * NP + p) is row p * RPT + r of column j), so blocks read and write whole lines
// whatever cut of the columns they have, and the cut changes no sum: the order of a row's sums depends on n alone.
#include "common.cuh"
#include <math.h>

// ---- the shifted mixes ------------------------------------------------------------------------------------------------
// x [T, d]; mu fp32 [M, d]; out [M][T, d] (matrix m at out + m * out_mat_stride); state fp32 [slots, state_stride] with
// the previous row at prev_off.
template <typename T>
__global__ void __launch_bounds__(256) shift_mix_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ mu,
    int M, T* __restrict__ out, long long out_mat_stride, float* __restrict__ state, long long state_stride, long long prev_off,
    const int* __restrict__ positions, const int* __restrict__ row_seq, const int* __restrict__ q_start,
    const int* __restrict__ slots, int num_seqs, int d, int* status) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int seq = row_seq[t];
  if (seq < 0 || seq >= num_seqs) {                  // a padding row of a fixed-shape step: finite values, nothing kept
    if (seq >= 0 && threadIdx.x == 0) set_status(status, SI_BAD_SEQ);
    for (int m = 0; m < M; ++m)
      for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < d; c += blockDim.x * gridDim.y)
        out[(size_t)m * out_mat_stride + (size_t)t * d + c] = from_f32<T>(0.f);
    return;
  }
  const int first_row = q_start[seq];
  const bool first = t == first_row;
  const int pos = positions[t];
  const T* xr = x + (size_t)t * x_stride;
  const T* xp = x + (size_t)(t - 1) * x_stride;
  float* keep = state + (size_t)slots[seq] * state_stride + prev_off;
  const T* xl = x + (size_t)(q_start[seq + 1] - 1) * x_stride;       // the portion's last row
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < d; c += blockDim.x * gridDim.y) {
    const float h = to_f32<T>(xr[c]);
    float prev;
    if (!first) prev = to_f32<T>(xp[c]);
    else {
      prev = pos > 0 ? keep[c] : 0.f;
      keep[c] = to_f32<T>(xl[c]);
    }
    const float diff = prev - h;
    for (int m = 0; m < M; ++m)
      out[(size_t)m * out_mat_stride + (size_t)t * d + c] = from_f32<T>(fmaf(diff, mu[(size_t)m * d + c], h));
  }
}

// The same, eight entries a thread with 16-byte loads and stores (d, the strides and prev_off multiples of 8 entries, every
// tensor 16-byte aligned).
template <typename T> struct TmVec8;
template <> struct TmVec8<float> {
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct TmVec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

template <typename T>
__global__ void __launch_bounds__(256) shift_mix_vec_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ mu,
    int M, T* __restrict__ out, long long out_mat_stride, float* __restrict__ state, long long state_stride, long long prev_off,
    const int* __restrict__ positions, const int* __restrict__ row_seq, const int* __restrict__ q_start,
    const int* __restrict__ slots, int num_seqs, int d, int* status) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int seq = row_seq[t];
  const int c_first = (blockIdx.y * blockDim.x + threadIdx.x) * 8, c_step = blockDim.x * gridDim.y * 8;
  if (seq < 0 || seq >= num_seqs) {                  // a padding row of a fixed-shape step: finite values, nothing kept
    if (seq >= 0 && threadIdx.x == 0) set_status(status, SI_BAD_SEQ);
    const float zero[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int m = 0; m < M; ++m)
      for (int c = c_first; c < d; c += c_step) TmVec8<T>::store(out + (size_t)m * out_mat_stride + (size_t)t * d + c, zero);
    return;
  }
  const bool first = t == q_start[seq];
  const int pos = positions[t];
  const T* xr = x + (size_t)t * x_stride;
  const T* xp = x + (size_t)(t - 1) * x_stride;
  float* keep = state + (size_t)slots[seq] * state_stride + prev_off;
  const T* xl = x + (size_t)(q_start[seq + 1] - 1) * x_stride;       // the portion's last row
  for (int c = c_first; c < d; c += c_step) {
    float h[8], prev[8], diff[8], w[8], o[8];
    TmVec8<T>::load(xr + c, h);
    if (!first) TmVec8<T>::load(xp + c, prev);
    else {
      if (pos > 0) TmVec8<float>::load(keep + c, prev);
      else {
#pragma unroll
        for (int e = 0; e < 8; ++e) prev[e] = 0.f;
      }
      float last[8];
      TmVec8<T>::load(xl + c, last);
      TmVec8<float>::store(keep + c, last);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) diff[e] = prev[e] - h[e];
    for (int m = 0; m < M; ++m) {
      TmVec8<float>::load(mu + (size_t)m * d + c, w);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = fmaf(diff[e], w[e], h[e]);
      TmVec8<T>::store(out + (size_t)m * out_mat_stride + (size_t)t * d + c, o);
    }
  }
}

SI_EXPORT int si_shift_mix(const void* x, int dtype, long long x_stride, const float* mu, int M, void* out,
                           long long out_mat_stride, float* state, long long state_stride, long long prev_off,
                           const int* positions, const int* row_seq, const int* q_start, const int* slots, int num_tokens,
                           int num_seqs, int d, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (M <= 0 || d <= 0 || prev_off < 0 || prev_off + d > state_stride) return -2;
  const uintptr_t all = (uintptr_t)x | (uintptr_t)mu | (uintptr_t)out | (uintptr_t)state;
  if (d % 8 == 0 && x_stride % 8 == 0 && out_mat_stride % 8 == 0 && state_stride % 8 == 0 && prev_off % 8 == 0 && (all & 15) == 0) {
    const dim3 vblock(d >= 2048 ? 256 : (d >= 1024 ? 128 : 64));
    const dim3 vgrid(num_tokens, si_row_shares(num_tokens, d / 8, vblock.x));
    if (dtype == SI_BF16)
      si_launch(shift_mix_vec_kernel<__nv_bfloat16>, vgrid, vblock, 0, stream, (const __nv_bfloat16*)x, x_stride, mu, M,
                (__nv_bfloat16*)out, out_mat_stride, state, state_stride, prev_off, positions, row_seq, q_start, slots, num_seqs,
                d, status);
    else
      si_launch(shift_mix_vec_kernel<float>, vgrid, vblock, 0, stream, (const float*)x, x_stride, mu, M, (float*)out,
                out_mat_stride, state, state_stride, prev_off, positions, row_seq, q_start, slots, num_seqs, d, status);
    return si_last_error();
  }
  const dim3 block(d >= 1024 ? 256 : 128);
  const dim3 grid(num_tokens, si_row_shares(num_tokens, d, block.x));
  if (dtype == SI_BF16)
    si_launch(shift_mix_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)x, x_stride, mu, M,
              (__nv_bfloat16*)out, out_mat_stride, state, state_stride, prev_off, positions, row_seq, q_start, slots, num_seqs,
              d, status);
  else
    si_launch(shift_mix_kernel<float>, grid, block, 0, stream, (const float*)x, x_stride, mu, M, (float*)out, out_mat_stride,
              state, state_stride, prev_off, positions, row_seq, q_start, slots, num_seqs, d, status);
  return si_last_error();
}

// ---- decay and fp32 copies ----------------------------------------------------------------------------------------------
// r, k, v: rows of C values each in the compute dtype; z [T, L] likewise; w2t fp32 [L, C] (the second low-rank matrix,
// transposed); w0 fp32 [C]; xs fp32 [T, 4C] = [r | k | v | decay]. A block takes ROWS rows and 256 channels (blockIdx.y),
// a thread one channel: it walks the L rows of w2t once for all its rows, in the order l = 0, 1, ... whatever ROWS is, so a
// row's decay does not depend on how many rows the step has.
template <typename T, int ROWS>
__global__ void __launch_bounds__(256) time_mix_prepare_kernel(const T* __restrict__ r, long long r_stride, const T* __restrict__ k,
    long long k_stride, const T* __restrict__ v, long long v_stride, const T* __restrict__ z, long long z_stride,
    const float* __restrict__ w2t, const float* __restrict__ w0, float* __restrict__ xs, int rows, int C, int L) {
  extern __shared__ float th[];                      // [L][ROWS]: tanh of the rows' low-rank values
  pdl_prologue();
  const int t0 = blockIdx.x * ROWS;
  for (int idx = threadIdx.x; idx < ROWS * L; idx += blockDim.x) {
    const int rr = idx / L, l = idx - rr * L;
    th[l * ROWS + rr] = t0 + rr < rows ? tanhf(to_f32<T>(z[(size_t)(t0 + rr) * z_stride + l])) : 0.f;
  }
  __syncthreads();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float acc[ROWS];
#pragma unroll
  for (int rr = 0; rr < ROWS; ++rr) acc[rr] = 0.f;
#pragma unroll(ROWS == 1 ? 16 : 4)             // a single row's walk is a chain of loads: many of them in flight
  for (int l = 0; l < L; ++l) {
    const float w = w2t[(size_t)l * C + c];
#pragma unroll
    for (int rr = 0; rr < ROWS; ++rr) acc[rr] = fmaf(w, th[l * ROWS + rr], acc[rr]);
  }
  const float b = w0[c];
#pragma unroll
  for (int rr = 0; rr < ROWS; ++rr) {
    const int t = t0 + rr;
    if (t >= rows) break;
    float* o = xs + (size_t)t * 4 * C;
    o[c] = to_f32<T>(r[(size_t)t * r_stride + c]);
    o[C + c] = to_f32<T>(k[(size_t)t * k_stride + c]);
    o[2 * C + c] = to_f32<T>(v[(size_t)t * v_stride + c]);
    o[3 * C + c] = expf(-expf(acc[rr] + b));
  }
}

template <typename T, int ROWS>
static void time_mix_prepare_launch(const void* r, long long r_stride, const void* k, long long k_stride, const void* v,
                                    long long v_stride, const void* z, long long z_stride, const float* w2t, const float* w0,
                                    float* xs, int rows, int C, int L, cudaStream_t stream) {
  const dim3 grid((rows + ROWS - 1) / ROWS, (C + 255) / 256), block(256);
  si_launch(time_mix_prepare_kernel<T, ROWS>, grid, block, (size_t)ROWS * L * sizeof(float), stream, (const T*)r, r_stride,
            (const T*)k, k_stride, (const T*)v, v_stride, (const T*)z, z_stride, w2t, w0, xs, rows, C, L);
}

SI_EXPORT int si_time_mix_prepare(const void* r, long long r_stride, const void* k, long long k_stride, const void* v,
                                  long long v_stride, const void* z, long long z_stride, int dtype, const float* w2t,
                                  const float* w0, float* xs, int rows, int C, int L, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (C <= 0 || L <= 0 || L > 2048 || (C + 255) / 256 > 65535) return -2;
  // few rows: a row a block, so that the blocks are many; many rows: 16 a block, so that w2t is read once for all of them
  const bool many = (long long)rows * ((C + 255) / 256) >= 16LL * 4 * si_sm_count();
#define PREP_LAUNCH(T)                                                                                              \
  if (many && L <= 768) time_mix_prepare_launch<T, 16>(r, r_stride, k, k_stride, v, v_stride, z, z_stride, w2t, w0, xs, rows, C, L, stream); \
  else if (many) time_mix_prepare_launch<T, 4>(r, r_stride, k, k_stride, v, v_stride, z, z_stride, w2t, w0, xs, rows, C, L, stream); \
  else time_mix_prepare_launch<T, 1>(r, r_stride, k, k_stride, v, v_stride, z, z_stride, w2t, w0, xs, rows, C, L, stream);
  if (dtype == SI_BF16) { PREP_LAUNCH(__nv_bfloat16) } else { PREP_LAUNCH(float) }
#undef PREP_LAUNCH
  return si_last_error();
}

// ---- the recurrence -----------------------------------------------------------------------------------------------------
#define DECAY_CHUNK 32

__device__ __forceinline__ void tm_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void tm_cp16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}

// Rows a thread (RPT, a multiple of 4) and parts a column (NP, a power of two up to 16, RPT * NP >= n). A column is
// spread over many lanes: a token's step is a chain of dependent instructions in every warp, so a thread keeps few rows
// and the warps are many (measured: 16 rows a thread and 4 lanes a column took 2.5 times as long as 4 and 16).
struct DecayShape { int rpt, np; };
static DecayShape decay_shape(int n) {
  DecayShape s;
  s.rpt = ((n + 15) / 16 + 3) / 4 * 4;
  int parts = 1;
  while (parts * s.rpt < n) parts *= 2;
  s.np = parts;
  return s;
}
// fp32 entries of one head's state in a slot
SI_EXPORT long long si_decay_state_floats(int n) {
  if (n <= 0 || n > 512) return -1;
  const DecayShape s = decay_shape(n);
  return (long long)s.rpt * s.np * n;
}

// xs fp32 [T, 4C] = [r | k | v | decay], C = H * n; u fp32 [H, n]; y fp32 [T, C]. Shared memory: two buffers of `chunk`
// tokens of [r: RPT * NP | k: RPT * NP | decay: RPT * NP | v: cols] (rows beyond n stay zero). A thread keeps its rows two
// by two (packed fp32 arithmetic): with t = k v_j, the read-out takes r (S + u t) and the state becomes w S + t, four
// packed operations for two rows.
template <int RPT, int NP>
__global__ void __launch_bounds__(256, RPT <= 8 ? 2 : 1) decay_scan_kernel(const float* __restrict__ xs, long long xs_stride,
    const float* __restrict__ u, float* __restrict__ state, long long state_stride, float* __restrict__ y, long long y_stride,
    const int* __restrict__ q_start, const int* __restrict__ ctx_len, const int* __restrict__ slots, int H, int n, int cols,
    int chunk) {
  extern __shared__ __align__(16) float sm[];
  pdl_prologue();
  const int s = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * cols;
  const int row0 = q_start[s], cnt = q_start[s + 1] - row0;
  if (cnt <= 0) return;
  const int pos0 = ctx_len[s] - cnt;
  const int p = threadIdx.x % NP, jl = threadIdx.x / NP;
  const int j = j0 + jl;
  const bool col_ok = jl < cols && j < n;
  const int C = H * n;
  float* S = state + (size_t)slots[s] * state_stride + (size_t)h * RPT * NP * n + (size_t)(col_ok ? j : 0) * NP + p;
  const size_t s_step = (size_t)n * NP;
  float2 st[RPT / 2], uu[RPT / 2];
#pragma unroll
  for (int r = 0; r < RPT / 2; ++r) {
    const bool have = col_ok && pos0 > 0;
    st[r].x = have ? S[(size_t)(2 * r) * s_step] : 0.f;
    st[r].y = have ? S[(size_t)(2 * r + 1) * s_step] : 0.f;
    const int i = p * RPT + 2 * r;
    uu[r].x = i < n ? u[(size_t)h * n + i] : 0.f;
    uu[r].y = i + 1 < n ? u[(size_t)h * n + i + 1] : 0.f;
  }
  const int dkp = RPT * NP;
  const int per_tok = 3 * dkp + ((cols + 3) & ~3);
  const int used = min(chunk, cnt) * per_tok;            // what of a buffer this launch's tokens reach (a decode row: one token)
  for (int idx = threadIdx.x; idx < 2 * used; idx += blockDim.x) sm[idx < used ? idx : chunk * per_tok + idx - used] = 0.f;
  __syncthreads();
  const size_t head_off = (size_t)h * n;
  const bool wide = n % 4 == 0 && xs_stride % 4 == 0 && ((uintptr_t)xs & 15) == 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int unit = wide ? 4 : 1;
  auto fetch = [&](int c0, int buf) {           // a token a warp; lanes walk a part's entries, 16 bytes each where aligned
    const int cn = min(chunk, cnt - c0);
    for (int tt = warp; tt < cn; tt += nwarps) {
      float* dst = sm + ((size_t)buf * chunk + tt) * per_tok;
      const float* row = xs + (size_t)(row0 + c0 + tt) * xs_stride + head_off;
#pragma unroll
      for (int part = 0; part < 3; ++part) {                                    // 0 r, 1 k, 2 decay
        const float* src = row + (size_t)(part == 2 ? 3 : part) * C;
        float* d = dst + part * dkp;
        for (int i = lane * unit; i < n; i += 32 * unit) {
          if (wide) tm_cp16(d + i, src + i);
          else tm_cp4(d + i, src + i);
        }
      }
      for (int e = lane; e < cols; e += 32)
        if (j0 + e < n) tm_cp4(dst + 3 * dkp + e, row + (size_t)2 * C + j0 + e);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  // Where rows are aligned and a token has at most 32 * DECAY_SLOTS pieces of 16 bytes (its r, k and decay of this head,
  // then this block's columns of v), every lane knows its pieces once and for all: where they lie in a row of xs and
  // where they go in a token's shared memory. A token's copy is then a few instructions.
  constexpr int DECAY_SLOTS = 4;
  const int pr = n / 4, pieces = 3 * pr + cols / 4;
  const bool quick = wide && cols % 4 == 0 && j0 + cols <= n && pieces <= 32 * DECAY_SLOTS && 4LL * C < (1LL << 30);
  int src_off[DECAY_SLOTS], dst_off[DECAY_SLOTS];
#pragma unroll
  for (int q = 0; q < DECAY_SLOTS; ++q) {
    const int idx = lane + 32 * q;
    src_off[q] = 0;
    dst_off[q] = -1;
    if (quick && idx < 3 * pr) {
      const int part = idx / pr, i = (idx - part * pr) * 4;
      src_off[q] = (part == 2 ? 3 : part) * C + i;
      dst_off[q] = part * dkp + i;
    } else if (quick && idx < pieces) {
      const int e = (idx - 3 * pr) * 4;
      src_off[q] = 2 * C + j0 + e;
      dst_off[q] = 3 * dkp + e;
    }
  }
  auto fetch_quick = [&](int c0, int buf) {
    const int cn = min(chunk, cnt - c0);
    for (int tt = warp; tt < cn; tt += nwarps) {
      float* dst = sm + ((size_t)buf * chunk + tt) * per_tok;
      const float* row = xs + (size_t)(row0 + c0 + tt) * xs_stride + head_off;
#pragma unroll
      for (int q = 0; q < DECAY_SLOTS; ++q)
        if (dst_off[q] >= 0) tm_cp16(dst + dst_off[q], row + src_off[q]);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  if (quick) fetch_quick(0, 0);
  else fetch(0, 0);
  int buf = 0;
  for (int c0 = 0; c0 < cnt; c0 += chunk, buf ^= 1) {
    const int cn = min(chunk, cnt - c0);
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();                            // this chunk has arrived, and everyone is done with the other buffer
    if (c0 + chunk < cnt) {
      if (quick) fetch_quick(c0 + chunk, buf ^ 1);
      else fetch(c0 + chunk, buf ^ 1);
    }
    const float* tok = sm + (size_t)buf * chunk * per_tok;
    float* yp = y + (size_t)(row0 + c0) * y_stride + head_off + j;
#pragma unroll(RPT <= 8 ? 4 : 2)               // tokens side by side: only the state's own update is a chain from token to token
    for (int tt = 0; tt < cn; ++tt, tok += per_tok, yp += y_stride) {
      const float4* r4 = reinterpret_cast<const float4*>(tok) + p * (RPT / 4);
      const float4* k4 = reinterpret_cast<const float4*>(tok + dkp) + p * (RPT / 4);
      const float4* w4 = reinterpret_cast<const float4*>(tok + 2 * dkp) + p * (RPT / 4);
      const float vj = col_ok ? tok[3 * dkp + jl] : 0.f;
      const float2 v2 = make_float2(vj, vj);
      float2 ra = make_float2(0.f, 0.f), rb = make_float2(0.f, 0.f);     // this thread's parts of r . (S + diag(u) k v^T)[:, j]
#pragma unroll
      for (int c = 0; c < RPT / 4; ++c) {
        const float4 rv = r4[c], kv = k4[c], wv = w4[c];
        const float2 t0 = __fmul2_rn(make_float2(kv.x, kv.y), v2), t1 = __fmul2_rn(make_float2(kv.z, kv.w), v2);
        ra = __ffma2_rn(make_float2(rv.x, rv.y), __ffma2_rn(uu[2 * c], t0, st[2 * c]), ra);
        rb = __ffma2_rn(make_float2(rv.z, rv.w), __ffma2_rn(uu[2 * c + 1], t1, st[2 * c + 1]), rb);
        st[2 * c] = __ffma2_rn(make_float2(wv.x, wv.y), st[2 * c], t0);
        st[2 * c + 1] = __ffma2_rn(make_float2(wv.z, wv.w), st[2 * c + 1], t1);
      }
      float o = (ra.x + ra.y) + (rb.x + rb.y);
#pragma unroll
      for (int off = 1; off < NP; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (p == 0 && col_ok) *yp = o;
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

SI_EXPORT int si_decay_scan(const float* xs, long long xs_stride, const float* u, float* state, long long state_stride,
                            float* y, long long y_stride, const int* q_start, const int* ctx_len, const int* slots,
                            int num_seqs, int H, int n, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (H <= 0 || H > 65535 || n <= 0 || n > 512) return -2;
  const DecayShape sh = decay_shape(n);
  if (sh.rpt * sh.np < n || state_stride < (long long)H * sh.rpt * sh.np * n) return -2;
  // columns a block: as many as 256 threads hold, fewer while the blocks do not fill the device (a block's tokens are a
  // chain of dependent steps, so more blocks of fewer columns finish sooner); never less than a warp
  int cols = 256 / sh.np;
  if (cols > n) cols = n;
  if (cols < 1) cols = 1;
  const long long per = (long long)num_seqs * H;
  while (cols > 1 && (cols / 2) * sh.np >= 32 && per * ((n + cols - 1) / cols) < si_sm_count()) cols /= 2;
  const int zb = (n + cols - 1) / cols;
  if (zb > 65535) return -2;
  const int threads = ((cols * sh.np + 31) / 32) * 32;
  // tokens a buffer: 32, fewer where two buffers of that many would not fit
  const size_t per_tok = (size_t)(3 * sh.np * sh.rpt + ((cols + 3) & ~3)) * sizeof(float);
  int chunk = DECAY_CHUNK;
  while (chunk > 1 && 2 * chunk * per_tok > 200 * 1024) chunk /= 2;
  const size_t smem = 2 * chunk * per_tok;
  if (smem > 200 * 1024) return -2;
  const dim3 grid(num_seqs, H, zb), block(threads);
#define DECAY_LAUNCH(R, P)                                                                                           \
  {                                                                                                                  \
    static size_t configured = 0;                                                                                    \
    if (smem > 48 * 1024 && smem > configured) {                                                                     \
      if (cudaFuncSetAttribute(decay_scan_kernel<R, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
        return -2;                                                                                                   \
      configured = smem;                                                                                             \
    }                                                                                                                \
    si_launch(decay_scan_kernel<R, P>, grid, block, smem, stream, xs, xs_stride, u, state, state_stride, y, y_stride, \
              q_start, ctx_len, slots, H, n, cols, chunk);                                                           \
  }
  if (sh.np < 16) {
    if (sh.rpt != 4) return -2;
    switch (sh.np) {
      case 1: DECAY_LAUNCH(4, 1) break;
      case 2: DECAY_LAUNCH(4, 2) break;
      case 4: DECAY_LAUNCH(4, 4) break;
      case 8: DECAY_LAUNCH(4, 8) break;
      default: return -2;
    }
  } else if (sh.np == 16) {
    switch (sh.rpt) {                        // n up to 512: up to 32 rows a thread
      case 4: DECAY_LAUNCH(4, 16) break;
      case 8: DECAY_LAUNCH(8, 16) break;
      case 12: DECAY_LAUNCH(12, 16) break;
      case 16: DECAY_LAUNCH(16, 16) break;
      case 20: DECAY_LAUNCH(20, 16) break;
      case 24: DECAY_LAUNCH(24, 16) break;
      case 28: DECAY_LAUNCH(28, 16) break;
      case 32: DECAY_LAUNCH(32, 16) break;
      default: return -2;
    }
  } else {
    return -2;
  }
#undef DECAY_LAUNCH
  return si_last_error();
}
