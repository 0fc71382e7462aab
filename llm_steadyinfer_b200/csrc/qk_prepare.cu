// What stands between a stacked q/k/v projection and attention over the paged cache when queries and keys are
// normalised per vector and rotated in part, and when several key vectors share one value vector:
//   row = [ q: NQ vectors of dk | k: NK vectors of dk | v: NV vectors of dv | ... ]
//   x  <- w * x * rsqrt(mean(x^2) + eps)          every q and k vector, w shared by all (w absent: no norm); or
//                                                 (`whole`) all q vectors of a row as one vector, and all its k vectors,
//                                                 with weights of that whole size
//   x  <- rotate(x)                               the first rd entries: pairs (2i, 2i + 1) ("interleaved") or
//                                                 (i, i + rd/2) ("halves"), angle pos * inv_freq[i], all in fp32:
//                                                 (u, v) -> (u c - v s, v c + u s), c = rot_scale cos a,
//                                                 s = rot_scale sin a; the rest pass
//   q into `q_out` (which may be the rows themselves); k into the key pages [pages, NK, page_size, dk]; v as it is
//   into the value pages [pages, NV, page_size, dv].
// With `maps` M > 1 the vectors of a head come as M maps, [head][map], and map m of a head reads key vector
// (key head, m): q_out is then ordered [key head][map][head of the group], so that query vector i reads key vector
// i / (NQ / NK) as in any grouped attention (q_out must not be the rows then).
// One block a token row, one warp a vector. The second kernel of the file combines the maps of a differential
// attention (see there).
#include "common.cuh"
#include <math.h>

// A lane takes pairs of entries: the two of a rotation where the vector is rotated, neighbours elsewhere. Every entry is
// read once, kept in registers over the warp's sum, and written once, so source and destination may be the same.
// ITEMS: pairs a lane (1, 2, 4 or 10: sizes up to 64, 128, 256, 640)
template <typename T, int ITEMS>
__device__ __forceinline__ void norm_rotate_vector(const T* __restrict__ src, T* __restrict__ dst, const float* __restrict__ w,
                                                   float eps, const float* __restrict__ sc_table, int rd, int interleaved,
                                                   int dk, int lane, float inv_given = -1.f) {
  const int half = rd / 2;
  const int items = interleaved ? (dk + 1) / 2 : half + (dk - rd + 1) / 2;
  float xa[ITEMS], xb[ITEMS];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < ITEMS; ++c) {
    const int t = lane + 32 * c;
    int ia, ib;
    if (interleaved) { ia = 2 * t; ib = ia + 1; }
    else if (t < half) { ia = t; ib = t + half; }
    else { ia = rd + 2 * (t - half); ib = ia + 1; }
    xa[c] = (t < items) ? to_f32<T>(src[ia]) : 0.f;
    xb[c] = (t < items && ib < dk) ? to_f32<T>(src[ib]) : 0.f;
    ss = fmaf(xa[c], xa[c], fmaf(xb[c], xb[c], ss));
  }
  // inv_given: the statistics are the caller's (a norm over more than this vector)
  const float inv = inv_given >= 0.f ? inv_given : (w ? rsqrtf(warp_sum(ss) / (float)dk + eps) : 1.f);
#pragma unroll
  for (int c = 0; c < ITEMS; ++c) {
    const int t = lane + 32 * c;
    if (t >= items) continue;
    int ia, ib, f;
    bool rot;
    if (interleaved) { ia = 2 * t; ib = ia + 1; f = t; rot = ia < rd; }
    else if (t < half) { ia = t; ib = t + half; f = t; rot = true; }
    else { ia = rd + 2 * (t - half); ib = ia + 1; f = 0; rot = false; }
    const bool has_b = ib < dk;
    float ya = xa[c] * inv * (w ? w[ia] : 1.f);
    float yb = has_b ? xb[c] * inv * (w ? w[ib] : 1.f) : 0.f;
    if (rot) {
      const float sn = sc_table[f], cs = sc_table[half + f];
      const float ra = ya * cs - yb * sn, rb = yb * cs + ya * sn;
      ya = ra; yb = rb;
    }
    dst[ia] = from_f32<T>(ya);
    if (has_b) dst[ib] = from_f32<T>(yb);
  }
}

template <typename T, int ITEMS>
__global__ void __launch_bounds__(256) qk_prepare_kernel(T* __restrict__ rows, long long row_stride, const float* __restrict__ q_w,
    const float* __restrict__ k_w, float eps, const float* __restrict__ inv_freq, int rd, int interleaved,
    const int* __restrict__ positions, const int* __restrict__ row_seq, const int* __restrict__ block_table, int table_width,
    T* __restrict__ k_cache, T* __restrict__ v_cache, int num_pages, int page_size, int num_seqs, int NQ, int NK, int NV,
    int dk, int dv, T* __restrict__ q_out, long long q_out_stride, int maps, int whole, float rot_scale, int* status) {
  extern __shared__ float sc_table[];                  // the row's sines, then its cosines: rd / 2 each, once for all vectors
  __shared__ float red[33];
  pdl_prologue();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int pos = positions[t];
  const int seq = row_seq[t];
  if (seq < 0) return;                               // a padding row of a fixed-shape step
  if (seq >= num_seqs) {
    if (threadIdx.x == 0) set_status(status, SI_BAD_SEQ);
    return;
  }
  long long page = -1;
  if (k_cache) {
    const int slot = pos / page_size;
    page = (pos >= 0 && slot < table_width) ? block_table[(size_t)seq * table_width + slot] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) set_status(status, SI_BAD_PAGE);
      page = -1;
    }
  }
  const int off = pos % page_size;
  T* row = rows + (size_t)t * row_stride;
  const float fpos = (float)pos;
  for (int f = threadIdx.x; f < rd / 2; f += blockDim.x) {
    float sn, cs;
    sincosf(fpos * inv_freq[f], &sn, &cs);
    sc_table[f] = sn * rot_scale;
    sc_table[rd / 2 + f] = cs * rot_scale;
  }
  float inv_q = -1.f, inv_k = -1.f;
  if (whole) {                                       // one norm over all of the row's q vectors, one over all its k vectors
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < NQ * dk; i += blockDim.x) { const float x = to_f32<T>(row[i]); sq = fmaf(x, x, sq); }
    for (int i = threadIdx.x; i < NK * dk; i += blockDim.x) { const float x = to_f32<T>(row[(size_t)NQ * dk + i]); sk = fmaf(x, x, sk); }
    inv_q = q_w ? rsqrtf(block_sum(sq, red) / (float)(NQ * dk) + eps) : 1.f;
    inv_k = k_w ? rsqrtf(block_sum(sk, red) / (float)(NK * dk) + eps) : 1.f;
  }
  __syncthreads();
  const int ratio = NQ / NK;                         // query vectors a key vector
  for (int vec = warp; vec < NQ + NK; vec += nwarps) {
    T* src = row + (size_t)vec * dk;
    if (vec < NQ) {
      const int head = vec / maps, m = vec - head * maps;
      const int place = ((head / ratio) * maps + m) * ratio + head % ratio;       // maps == 1: vec itself
      norm_rotate_vector<T, ITEMS>(src, q_out + (size_t)t * q_out_stride + (size_t)place * dk,
                            (whole && q_w) ? q_w + (size_t)vec * dk : q_w, eps, sc_table, rd, interleaved, dk, lane, inv_q);
    } else if (page >= 0) {
      T* dst = k_cache + (((size_t)page * NK + (vec - NQ)) * page_size + off) * dk;
      norm_rotate_vector<T, ITEMS>(src, dst, (whole && k_w) ? k_w + (size_t)(vec - NQ) * dk : k_w, eps, sc_table, rd, interleaved,
                            dk, lane, inv_k);
    }
  }
  if (page >= 0 && v_cache) {
    const T* vrow = row + (size_t)(NQ + NK) * dk;
    for (int idx = threadIdx.x; idx < NV * dv; idx += blockDim.x) {
      const int g = idx / dv, c = idx % dv;
      v_cache[(((size_t)page * NV + g) * page_size + off) * dv + c] = vrow[idx];
    }
  }
}

SI_EXPORT int si_qk_prepare(void* rows, int dtype, long long row_stride, const float* q_w, const float* k_w, float eps,
                            const float* inv_freq, int rd, int interleaved, const int* positions, const int* row_seq,
                            const int* block_table, int table_width, void* k_cache, void* v_cache, int num_pages,
                            int page_size, int num_tokens, int num_seqs, int NQ, int NK, int NV, int dk, int dv, void* q_out,
                            long long q_out_stride, int maps, int whole, float rot_scale, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (whole && maps != 1) return -2;
  if (dk <= 0 || dk > 640 || rd < 0 || rd > dk || rd % 2 || (rd > 0 && !inv_freq)) return -2;
  if (maps < 1 || NK <= 0 || NQ % NK || NK % maps || (maps > 1 && q_out == rows)) return -2;
  const size_t smem = (size_t)(rd > 0 ? rd : 1) * sizeof(float);
  // a warp a vector at a time; eight warps where there are vectors for them, so that a row's loads are in flight together
  const dim3 grid(num_tokens), block(NQ + NK >= 8 ? 256 : 128);
#define QK_LAUNCH(T, ITEMS)                                                                                              \
  si_launch(qk_prepare_kernel<T, ITEMS>, grid, block, smem, stream, (T*)rows, row_stride, q_w, k_w, eps, inv_freq, rd,      \
            interleaved, positions, row_seq, block_table, table_width, (T*)k_cache, (T*)v_cache, num_pages, page_size,   \
            num_seqs, NQ, NK, NV, dk, dv, (T*)q_out, q_out_stride, maps, whole, rot_scale, status)
  if (dtype == SI_BF16) {
    if (dk <= 64) QK_LAUNCH(__nv_bfloat16, 1);
    else if (dk <= 128) QK_LAUNCH(__nv_bfloat16, 2);
    else if (dk <= 256) QK_LAUNCH(__nv_bfloat16, 4);
    else QK_LAUNCH(__nv_bfloat16, 10);
  } else {
    if (dk <= 64) QK_LAUNCH(float, 1);
    else if (dk <= 128) QK_LAUNCH(float, 2);
    else if (dk <= 256) QK_LAUNCH(float, 4);
    else QK_LAUNCH(float, 10);
  }
#undef QK_LAUNCH
  return si_last_error();
}

// ---- the maps of a differential attention into one head ------------------------------------------------------------
//   a[t, g, m, hl]: the maps' results (dv each, fp32 or the compute dtype) in the order the prepared queries have:
//   key head g, map m, head hl of the group (`ratio` heads a key head); head h = g * ratio + hl
//   o = a0 - lambda * a1;   o <- o * rsqrt(mean(o^2) + eps) * post;   o <- o * sigmoid(gate[t, h])   (gate absent: none)
// One warp a (row, head); everything in fp32.
template <typename TA, typename T>
__global__ void __launch_bounds__(256) diff_combine_kernel(const TA* __restrict__ a, long long a_stride, const T* __restrict__ gate,
    long long gate_stride, T* __restrict__ out, long long out_stride, long long pairs, int H, int dv, int ratio, float lambda,
    float eps, float post) {
  pdl_prologue();
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= pairs) return;
  const int lane = threadIdx.x & 31;
  const long long t = w / H;
  const int h = (int)(w - t * H);
  const TA* a0 = a + t * a_stride + ((size_t)(h / ratio) * 2 * ratio + h % ratio) * dv;
  const TA* a1 = a0 + (size_t)ratio * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) {
    const float o = to_f32<TA>(a0[i]) - lambda * to_f32<TA>(a1[i]);
    ss += o * o;
  }
  ss = warp_sum(ss);
  float f = rsqrtf(ss / (float)dv + eps) * post;
  if (gate) f *= 1.f / (1.f + expf(-to_f32<T>(gate[t * gate_stride + h])));
  T* o = out + t * out_stride + (size_t)h * dv;
  for (int i = lane; i < dv; i += 32) o[i] = from_f32<T>((to_f32<TA>(a0[i]) - lambda * to_f32<TA>(a1[i])) * f);
}

SI_EXPORT int si_diff_combine(const void* a, int a_dtype, long long a_stride, const void* gate, long long gate_stride, void* out,
                              int dtype, long long out_stride, int rows, int H, int dv, int ratio, float lambda, float eps,
                              float post, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || dv <= 0 || ratio <= 0 || H % ratio) return -2;
  const long long pairs = (long long)rows * H;
  const dim3 grid((unsigned)((pairs + 7) / 8)), block(256);
  if (dtype == SI_BF16 && a_dtype == SI_F32)
    si_launch(diff_combine_kernel<float, __nv_bfloat16>, grid, block, 0, stream, (const float*)a, a_stride,
              (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, out_stride, pairs, H, dv, ratio, lambda, eps, post);
  else if (dtype == SI_BF16 && a_dtype == SI_BF16)
    si_launch(diff_combine_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)a, a_stride,
              (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, out_stride, pairs, H, dv, ratio, lambda, eps, post);
  else if (dtype == SI_F32 && a_dtype == SI_F32)
    si_launch(diff_combine_kernel<float, float>, grid, block, 0, stream, (const float*)a, a_stride, (const float*)gate,
              gate_stride, (float*)out, out_stride, pairs, H, dv, ratio, lambda, eps, post);
  else
    return -2;
  return si_last_error();
}

// ---- attention weights mixed over the heads ("talking heads" behind the softmax) ---------------------------------------
// Mixing the heads' weights, w'_h(i, j) = sum_g talk[h, g] w_g(i, j), and applying w'_h to the values of head h's own
// key/value head is the same as mixing what every head's weights give on those values:
//   out_h = sum_g talk[h, g] * a[g, kv(h)],      a[g, c] = sum_j w_g(i, j) v_c(j)
// so attention runs with every query head over the values of all G key/value heads side by side (one value "head" of
// G * dv entries), and this kernel forms the sums, multiplies by sigmoid(gate) and by `post`:
//   a [T, H, G * dv] (fp32 or the compute dtype), talk fp32 [H, H], gate [T, H * dv] (absent: none), out [T, H * dv].
// A block takes a row and a share of its entries (blockIdx.y: few rows still fill the device); everything in fp32.
template <typename TA, typename T>
__global__ void __launch_bounds__(256) talk_combine_kernel(const TA* __restrict__ a, long long a_stride, const float* __restrict__ talk,
    const T* __restrict__ gate, long long gate_stride, T* __restrict__ out, long long out_stride, int H, int G, int dv, float post) {
  extern __shared__ float tk[];                        // talk [H, H]
  pdl_prologue();
  for (int i = threadIdx.x; i < H * H; i += blockDim.x) tk[i] = talk[i];
  __syncthreads();
  const long long t = blockIdx.x;
  const TA* ar = a + t * a_stride;
  const int ratio = H / G, wide = G * dv;
  for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < H * dv; e += blockDim.x * gridDim.y) {
    const int h = e / dv, i = e - h * dv;
    const TA* col = ar + (size_t)(h / ratio) * dv + i;
    const float* th = tk + (size_t)h * H;
    float acc = 0.f;
    for (int g = 0; g < H; ++g) acc = fmaf(th[g], to_f32<TA>(col[(size_t)g * wide]), acc);
    acc *= post;
    if (gate) acc *= 1.f / (1.f + expf(-to_f32<T>(gate[t * gate_stride + e])));
    out[t * out_stride + e] = from_f32<T>(acc);
  }
}

SI_EXPORT int si_talk_combine(const void* a, int a_dtype, long long a_stride, const float* talk, const void* gate,
                              long long gate_stride, void* out, int dtype, long long out_stride, int rows, int H, int G, int dv,
                              float post, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || dv <= 0 || H > 100) return -2;
  const dim3 block(H * dv >= 1024 ? 256 : 128);
  const dim3 grid(rows, si_row_shares(rows, H * dv, block.x));
  const size_t smem = (size_t)H * H * sizeof(float);
  if (dtype == SI_BF16 && a_dtype == SI_F32)
    si_launch(talk_combine_kernel<float, __nv_bfloat16>, grid, block, smem, stream, (const float*)a, a_stride, talk,
              (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, out_stride, H, G, dv, post);
  else if (dtype == SI_BF16 && a_dtype == SI_BF16)
    si_launch(talk_combine_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, smem, stream, (const __nv_bfloat16*)a, a_stride, talk,
              (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, out_stride, H, G, dv, post);
  else if (dtype == SI_F32 && a_dtype == SI_F32)
    si_launch(talk_combine_kernel<float, float>, grid, block, smem, stream, (const float*)a, a_stride, talk, (const float*)gate,
              gate_stride, (float*)out, out_stride, H, G, dv, post);
  else
    return -2;
  return si_last_error();
}
