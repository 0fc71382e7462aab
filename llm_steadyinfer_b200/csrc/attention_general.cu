// Attention over the paged cache in its general form, fp32 arithmetic for fp32 or bf16 storage: the
// 32-bit path of every attention mixer and the yardstick of the tensor-core kernels of this form
// (attention_flex.cu). Beyond attention_ref.cu it takes
//   * a key size dk and a value size dv that differ,
//   * values that are the first dv entries of the keys (v_cache == nullptr: a latent that serves as both),
//   * a bias by distance: bias[min(i - j, nd - 1), head] (fp32 table [nd, H]) added to the scaled score,
//   * a sink per head: exp(sink[h]) joins the softmax denominator once, with no key and no value,
//   * a penalty in proportion to the distance: slope[h] * (i - j) taken off the scaled score (fp32 [H]),
//   * a query temperature by position: the scale of row i is multiplied by 1 + coef * ln(floor((i + 1) / every) + 1),
//   * an output gate: the result's entry (row, head, d) is multiplied by sigmoid(gate[row, head * dv + d]),
//   * a soft limit on the scaled score: s <- softcap * tanh(s / softcap) (before the bias),
//   * key heads that share a value head: `v_share` neighbouring key heads read one value head (the cache then holds
//     KV / v_share value heads), as the maps of a differential attention do,
//   * results in fp32 whatever the storage (out_f32), for a caller that goes on subtracting them.
//     s_j = scale * q_h . K[j, g] + bias[min(pos - j, nd - 1), h],  j in [max(0, pos - window + 1), pos]
//     out_h = sum_j exp(s_j) V[j, g] / (sum_j exp(s_j) + exp(sink_h))
// One block per (token row, query head); warp w of 4 walks keys j0 + w, j0 + w + 4, ... with a running
// maximum, the four partial results are merged at the end, so the order of a row's sums depends on its
// position alone. The file also holds the two kernels that put a step's keys and values into the pages for
// mixers that do not rotate them with rope_kv.cu: a plain store with dk != dv, and the latent form (norm of
// the latent, rotation of the shared key part and of the queries' rotated parts).
#include "common.cuh"
#include <math.h>

#define GEN_WARPS 4
#define GEN_MAX_PER_LANE 20   // key and value sizes up to 640
#define GEN_WIDE_PER_LANE 32  // a second instance for sizes up to 1,024 (a value head that holds several heads side by side)

template <typename T, typename TO, int PL = GEN_MAX_PER_LANE>
__global__ void __launch_bounds__(GEN_WARPS * 32)
attention_general_kernel(const T* __restrict__ q, long long q_row_stride,
                         const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                         const int* __restrict__ block_table, int table_width,
                         const int* __restrict__ row_seq, const int* __restrict__ positions,
                         TO* __restrict__ out, long long out_row_stride, int num_pages,
                         int page_size, int num_seqs, int H, int KV, int dk, int dv, float scale,
                         int window, const float* __restrict__ dist_bias, int nd,
                         const float* __restrict__ sink, float softcap, int v_share,
                         const float* __restrict__ slopes, float qt_coef, int qt_every,
                         const T* __restrict__ gate, long long gate_row_stride, int* status) {
  extern __shared__ float smem[];   // [GEN_WARPS][dv] accumulators, then m[GEN_WARPS], l[GEN_WARPS]
  const int t = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = h / (H / KV);
  const int pos = positions[t];
  const int seq = row_seq[t];
  TO* o = out + (size_t)t * out_row_stride + (size_t)h * dv;
  if (seq < 0 || seq >= num_seqs) {      // seq < 0 marks a padding row of a fixed-shape step
    if (threadIdx.x == 0 && seq >= 0) set_status(status, SI_BAD_SEQ);
    for (int d = threadIdx.x; d < dv; d += blockDim.x) o[d] = from_f32<TO>(0.f);
    return;
  }
  const int* table = block_table + (size_t)seq * table_width;
  const T* qh = q + (size_t)t * q_row_stride + (size_t)h * dk;
  const size_t v_stride = v_cache ? dv : dk;
  const T* vbase = v_cache ? v_cache : k_cache;

  float qr[PL], acc[PL];
#pragma unroll
  for (int i = 0; i < PL; ++i) {
    const int d = lane + 32 * i;
    qr[i] = d < dk ? to_f32<T>(qh[d]) : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  if (qt_every > 0) scale *= 1.f + qt_coef * logf((float)((pos + 1) / qt_every + 1));
  const float slope = slopes ? slopes[h] : 0.f;
  const int j0 = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  for (int j = j0 + warp; j <= pos; j += GEN_WARPS) {
    const int slot = j / page_size;
    const int page = slot < table_width ? table[slot] : -1;
    if (page < 0 || page >= num_pages) {
      if (lane == 0) set_status(status, SI_BAD_PAGE);
      continue;
    }
    const size_t tok = ((size_t)page * KV + g) * page_size + (j - slot * page_size);
    const T* kp = k_cache + tok * dk;
    const T* vp = vbase + (v_share > 1 ? ((size_t)page * (KV / v_share) + g / v_share) * page_size + (j - slot * page_size)
                                       : tok) * v_stride;
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < PL; ++i) {
      const int d = lane + 32 * i;
      if (d < dk) dot += qr[i] * to_f32<T>(kp[d]);
    }
    dot = warp_sum(dot) * scale;
    if (softcap > 0.f) dot = softcap * tanhf(dot / softcap);
    if (dist_bias) dot += dist_bias[(size_t)min(pos - j, nd - 1) * H + h];
    dot -= slope * (float)(pos - j);
    const float m_new = fmaxf(m, dot);
    const float corr = expf(m - m_new);
    const float p = expf(dot - m_new);
    l = l * corr + p;
#pragma unroll
    for (int i = 0; i < PL; ++i) {
      const int d = lane + 32 * i;
      if (d < dv) acc[i] = acc[i] * corr + p * to_f32<T>(vp[d]);
    }
    m = m_new;
  }
  float* sacc = smem;
  float* sm = smem + GEN_WARPS * dv;
  float* sl = sm + GEN_WARPS;
#pragma unroll
  for (int i = 0; i < PL; ++i) {
    const int d = lane + 32 * i;
    if (d < dv) sacc[warp * dv + d] = acc[i];
  }
  if (lane == 0) { sm[warp] = m; sl[warp] = l; }
  __syncthreads();
  float M = sink ? sink[h] : -INFINITY;
#pragma unroll
  for (int w = 0; w < GEN_WARPS; ++w) M = fmaxf(M, sm[w]);
  float L = sink ? expf(sink[h] - M) : 0.f, wgt[GEN_WARPS];
#pragma unroll
  for (int w = 0; w < GEN_WARPS; ++w) {
    wgt[w] = sm[w] == -INFINITY ? 0.f : expf(sm[w] - M);
    L += sl[w] * wgt[w];
  }
  for (int d = threadIdx.x; d < dv; d += blockDim.x) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < GEN_WARPS; ++w) v += sacc[w * dv + d] * wgt[w];
    v = L > 0.f ? v / L : 0.f;
    if (gate) v /= 1.f + expf(-to_f32<T>(gate[(size_t)t * gate_row_stride + (size_t)h * dv + d]));
    o[d] = from_f32<TO>(v);
  }
}

SI_EXPORT int si_attention_general(const void* q, int dtype, long long q_row_stride, const void* k_cache,
                                   const void* v_cache, const int* block_table, int table_width,
                                   const int* row_seq, const int* positions, void* out,
                                   long long out_row_stride, int num_pages, int page_size, int num_tokens,
                                   int num_seqs, int H, int KV, int dk, int dv, float scale, int window,
                                   const float* dist_bias, int nd, const float* sink, float softcap, int v_share,
                                   int out_f32, const float* slopes, float qt_coef, int qt_every, const void* gate,
                                   long long gate_row_stride, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (dk > 32 * GEN_WIDE_PER_LANE || dv > 32 * GEN_WIDE_PER_LANE || dk <= 0 || dv <= 0 || KV <= 0 || H % KV) return -2;
  if (!v_cache && dv > dk) return -2;
  if (v_share < 1 || KV % v_share || (v_share > 1 && !v_cache)) return -2;
  if (dist_bias && nd <= 0) return -2;
  if (qt_every < 0) return -2;
  dim3 grid(num_tokens, H);
  const size_t smem = (size_t)(GEN_WARPS * dv + 2 * GEN_WARPS) * sizeof(float);
#define GEN_LAUNCH(T, TO, PL)                                                                                          \
  attention_general_kernel<T, TO, PL><<<grid, GEN_WARPS * 32, smem, stream>>>(                                         \
      (const T*)q, q_row_stride, (const T*)k_cache, (const T*)v_cache, block_table, table_width, row_seq, positions,   \
      (TO*)out, out_row_stride, num_pages, page_size, num_seqs, H, KV, dk, dv, scale, window, dist_bias, nd, sink,     \
      softcap, v_share, slopes, qt_coef, qt_every, (const T*)gate, gate_row_stride, status)
  if (dk > 32 * GEN_MAX_PER_LANE || dv > 32 * GEN_MAX_PER_LANE) {        // sizes above 640: the kernel with more entries a lane
    if (dtype == SI_BF16 && out_f32) GEN_LAUNCH(__nv_bfloat16, float, GEN_WIDE_PER_LANE);
    else if (dtype == SI_BF16) GEN_LAUNCH(__nv_bfloat16, __nv_bfloat16, GEN_WIDE_PER_LANE);
    else GEN_LAUNCH(float, float, GEN_WIDE_PER_LANE);
    return si_last_error();
  }
  if (dtype == SI_BF16 && out_f32) GEN_LAUNCH(__nv_bfloat16, float, GEN_MAX_PER_LANE);
  else if (dtype == SI_BF16) GEN_LAUNCH(__nv_bfloat16, __nv_bfloat16, GEN_MAX_PER_LANE);
  else GEN_LAUNCH(float, float, GEN_MAX_PER_LANE);
#undef GEN_LAUNCH
  return si_last_error();
}

// ---- stores into the pages -----------------------------------------------------------------------

// The page of (seq, pos), or -1 (with the status word set where that is a fault and not padding).
__device__ __forceinline__ long long page_of(const int* block_table, int table_width, int num_pages,
                                             int page_size, int num_seqs, int seq, int pos, int* status) {
  if (seq < 0) return -1;
  if (seq >= num_seqs) {
    if (threadIdx.x == 0) set_status(status, SI_BAD_SEQ);
    return -1;
  }
  const int slot = pos / page_size;
  const int p = (pos >= 0 && slot < table_width) ? block_table[(size_t)seq * table_width + slot] : -1;
  if (p < 0 || p >= num_pages) {
    if (threadIdx.x == 0) set_status(status, SI_BAD_PAGE);
    return -1;
  }
  return p;
}

// row = [ q: H*dk | k: KV*dk | v: KV*dv ]: k and v of every row go to their page as they are.
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ qkv, long long row_stride, const int* __restrict__ positions,
                                const int* __restrict__ row_seq, const int* __restrict__ block_table,
                                int table_width, T* __restrict__ k_cache, T* __restrict__ v_cache, int num_pages,
                                int page_size, int num_seqs, int H, int KV, int dk, int dv, int* status) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const long long page = page_of(block_table, table_width, num_pages, page_size, num_seqs, row_seq[t], pos, status);
  if (page < 0) return;
  const int off = pos % page_size;
  const T* krow = qkv + (size_t)t * row_stride + (size_t)H * dk;
  const T* vrow = krow + (size_t)KV * dk;
  for (int idx = threadIdx.x; idx < KV * dk; idx += blockDim.x) {
    const int g = idx / dk, c = idx % dk;
    k_cache[(((size_t)page * KV + g) * page_size + off) * dk + c] = krow[idx];
  }
  for (int idx = threadIdx.x; idx < KV * dv; idx += blockDim.x) {
    const int g = idx / dv, c = idx % dv;
    v_cache[(((size_t)page * KV + g) * page_size + off) * dv + c] = vrow[idx];
  }
}

SI_EXPORT int si_kv_store(const void* qkv, int dtype, long long row_stride, const int* positions, const int* row_seq,
                          const int* block_table, int table_width, void* k_cache, void* v_cache, int num_pages,
                          int page_size, int num_tokens, int num_seqs, int H, int KV, int dk, int dv, int* status,
                          cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (dtype == SI_BF16)
    si_launch(kv_store_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), 0, stream, (const __nv_bfloat16*)qkv,
              row_stride, positions, row_seq, block_table, table_width, (__nv_bfloat16*)k_cache,
              (__nv_bfloat16*)v_cache, num_pages, page_size, num_seqs, H, KV, dk, dv, status);
  else
    si_launch(kv_store_kernel<float>, dim3(num_tokens), dim3(128), 0, stream, (const float*)qkv, row_stride,
              positions, row_seq, block_table, table_width, (float*)k_cache, (float*)v_cache, num_pages,
              page_size, num_seqs, H, KV, dk, dv, status);
  return si_last_error();
}

// The latent form. Per row:
//   kv = [ latent: rk | shared key part: dr ]  (row of the down projection)
//   page[pos] = [ latent / sqrt(mean(latent^2) + eps) * w | rotate(shared part) ]         (one key "head" of rk + dr)
//   q_full[h] = [ (left as it is: the absorbed plain part, rk) | rotate(q[h, dq:dq + dr]) ]   for every head
//   q_exp[h]  = [ q[h, :dq] | rotate(q[h, dq:dq + dr]) ]                                       (optional)
// rotate(): the first rd of the dr entries in pairs (i, i + rd/2), or (2i, 2i + 1) when `interleaved`, angle
// pos * inv_freq[i] in fp32, cosine and sine times `rot_scale`; the other dr - rd entries pass.
__device__ __forceinline__ float rotated_entry(float u, float v, bool second, float angle, float rot_scale) {
  float s, c;
  sincosf(angle, &s, &c);
  s *= rot_scale; c *= rot_scale;
  return second ? v * c + u * s : u * c - v * s;
}
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ kv, long long kv_stride, const T* __restrict__ q,
                                      long long q_stride, T* __restrict__ q_full, long long qf_stride,
                                      T* __restrict__ q_exp, long long qe_stride, const float* __restrict__ norm_w, float eps, const float* __restrict__ inv_freq,
                                      int rd, const int* __restrict__ positions, const int* __restrict__ row_seq,
                                      const int* __restrict__ block_table, int table_width, T* __restrict__ k_cache,
                                      int num_pages, int page_size, int num_seqs, int H, int dq, int dr, int rk,
                                      int interleaved, float rot_scale, int* status) {
  __shared__ float red[33];
  pdl_prologue();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int seq = row_seq[t];
  const int half = rd / 2;
  const float fpos = (float)pos;
  // the queries' rotated parts
  const T* qrow = q + (size_t)t * q_stride;
  T* qf = q_full + (size_t)t * qf_stride;
  for (int idx = threadIdx.x; idx < H * dr; idx += blockDim.x) {
    const int h = idx / dr, i = idx % dr;
    const T* src = qrow + (size_t)h * (dq + dr) + dq;
    float y;
    if (i < rd) {
      const int f = interleaved ? i >> 1 : (i < half ? i : i - half);
      const int iu = interleaved ? 2 * f : f, iv = interleaved ? 2 * f + 1 : f + half;
      y = rotated_entry(to_f32<T>(src[iu]), to_f32<T>(src[iv]), i == iv, fpos * inv_freq[f], rot_scale);
    } else {
      y = to_f32<T>(src[i]);
    }
    qf[(size_t)h * (rk + dr) + rk + i] = from_f32<T>(y);
    if (q_exp) q_exp[(size_t)t * qe_stride + (size_t)h * (dq + dr) + dq + i] = from_f32<T>(y);
  }
  if (q_exp)                                   // the queries whole, for attention against keys that are expanded per head
    for (int idx = threadIdx.x; idx < H * dq; idx += blockDim.x) {
      const int h = idx / dq, i = idx % dq;
      q_exp[(size_t)t * qe_stride + (size_t)h * (dq + dr) + i] = qrow[(size_t)h * (dq + dr) + i];
    }
  if (!k_cache) return;
  const T* row = kv + (size_t)t * kv_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rk; i += blockDim.x) {
    const float x = to_f32<T>(row[i]);
    ss += x * x;
  }
  ss = block_sum(ss, red);
  const long long page = page_of(block_table, table_width, num_pages, page_size, num_seqs, seq, pos, status);
  if (page < 0) return;
  T* dst = k_cache + ((size_t)page * page_size + pos % page_size) * (rk + dr);
  const float rs = 1.f / sqrtf(ss / (float)rk + eps);
  for (int i = threadIdx.x; i < rk; i += blockDim.x) dst[i] = from_f32<T>(to_f32<T>(row[i]) * rs * norm_w[i]);
  for (int i = threadIdx.x; i < dr; i += blockDim.x) {
    float y;
    if (i < rd) {
      const int f = interleaved ? i >> 1 : (i < half ? i : i - half);
      const int iu = interleaved ? 2 * f : f, iv = interleaved ? 2 * f + 1 : f + half;
      y = rotated_entry(to_f32<T>(row[rk + iu]), to_f32<T>(row[rk + iv]), i == iv, fpos * inv_freq[f], rot_scale);
    } else {
      y = to_f32<T>(row[rk + i]);
    }
    dst[rk + i] = from_f32<T>(y);
  }
}

SI_EXPORT int si_latent_prepare(const void* kv, int dtype, long long kv_stride, const void* q, long long q_stride,
                                void* q_full, long long qf_stride, void* q_exp, long long qe_stride,
                                const float* norm_w, float eps,
                                const float* inv_freq, int rd, const int* positions, const int* row_seq,
                                const int* block_table, int table_width, void* k_cache, int num_pages, int page_size,
                                int num_tokens, int num_seqs, int H, int dq, int dr, int rk, int interleaved,
                                float rot_scale, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (rd < 0 || rd > dr || rd % 2) return -2;
  if (dtype == SI_BF16)
    si_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), 0, stream, (const __nv_bfloat16*)kv,
              kv_stride, (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)q_full, qf_stride, (__nv_bfloat16*)q_exp,
              qe_stride, norm_w, eps, inv_freq,
              rd, positions, row_seq, block_table, table_width, (__nv_bfloat16*)k_cache, num_pages, page_size,
              num_seqs, H, dq, dr, rk, interleaved, rot_scale, status);
  else
    si_launch(latent_prepare_kernel<float>, dim3(num_tokens), dim3(128), 0, stream, (const float*)kv, kv_stride,
              (const float*)q, q_stride, (float*)q_full, qf_stride, (float*)q_exp, qe_stride, norm_w, eps, inv_freq, rd,
              positions, row_seq,
              block_table, table_width, (float*)k_cache, num_pages, page_size, num_seqs, H, dq, dr, rk, interleaved,
              rot_scale, status);
  return si_last_error();
}

// ---- the latent form expanded for long prompt portions -------------------------------------------------------
// For the sequences listed in `seqs` ([E, 4] rows of (sequence of the step, first dense row, keys, first position)), the cached
// [latent | shared key part] rows of positions first .. first + keys - 1 are copied out of the pages into consecutive dense rows,
// where a matrix product can expand them into keys and values per head. One block per 8 keys of a sequence.
template <typename T>
__global__ void latent_gather_kernel(const T* __restrict__ k_cache, const int* __restrict__ block_table, int table_width,
                                     const int* __restrict__ seqs, T* __restrict__ dense, int num_pages, int page_size,
                                     int num_seqs, int width, int* status) {
  pdl_prologue();
  const int e = blockIdx.y;
  const int seq = seqs[4 * e], row0 = seqs[4 * e + 1], keys = seqs[4 * e + 2], first = seqs[4 * e + 3];
  for (int j = blockIdx.x * 8; j < min(keys, blockIdx.x * 8 + 8); ++j) {
    const long long page = page_of(block_table, table_width, num_pages, page_size, num_seqs, seq, first + j, status);
    if (page < 0) continue;
    const T* src = k_cache + ((size_t)page * page_size + (first + j) % page_size) * width;
    T* dst = dense + (size_t)(row0 + j) * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
  }
}

SI_EXPORT int si_latent_gather(const void* k_cache, int dtype, const int* block_table, int table_width, const int* seqs,
                               int num_listed, int max_keys, void* dense, int num_pages, int page_size, int num_seqs,
                               int width, int* status, cudaStream_t stream) {
  if (num_listed <= 0 || max_keys <= 0) return 0;
  if (num_listed > 65535) return -2;
  dim3 grid((max_keys + 7) / 8, num_listed);
  if (dtype == SI_BF16)
    si_launch(latent_gather_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)k_cache, block_table,
              table_width, seqs, (__nv_bfloat16*)dense, num_pages, page_size, num_seqs, width, status);
  else
    si_launch(latent_gather_kernel<float>, grid, dim3(128), 0, stream, (const float*)k_cache, block_table, table_width, seqs,
              (float*)dense, num_pages, page_size, num_seqs, width, status);
  return si_last_error();
}

// keys[t, h, :] = [ plain[t, h*dq : (h+1)*dq] | dense[t, rk : rk + dr] ]: every head's expanded plain key part beside the
// one rotated part that all heads share.
template <typename T>
__global__ void latent_expand_keys_kernel(const T* __restrict__ plain, const T* __restrict__ dense, T* __restrict__ keys,
                                          int H, int dq, int dr, int rk) {
  pdl_prologue();
  const size_t t = blockIdx.x;
  const int dk = dq + dr;
  for (int idx = threadIdx.x; idx < H * dk; idx += blockDim.x) {
    const int h = idx / dk, i = idx % dk;
    keys[t * H * dk + idx] = i < dq ? plain[t * H * dq + (size_t)h * dq + i] : dense[t * (rk + dr) + rk + (i - dq)];
  }
}

SI_EXPORT int si_latent_expand_keys(const void* plain, const void* dense, void* keys, int dtype, int rows, int H, int dq,
                                    int dr, int rk, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype == SI_BF16)
    si_launch(latent_expand_keys_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, (const __nv_bfloat16*)plain,
              (const __nv_bfloat16*)dense, (__nv_bfloat16*)keys, H, dq, dr, rk);
  else
    si_launch(latent_expand_keys_kernel<float>, dim3(rows), dim3(256), 0, stream, (const float*)plain, (const float*)dense,
              (float*)keys, H, dq, dr, rk);
  return si_last_error();
}
